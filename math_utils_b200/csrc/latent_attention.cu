// Rotary positions (rotate-half layout, any frequency table) and attention over a cache of latent rows.
//
// A latent row cache keeps ONE row per position, shared by all heads: `kv_rank` latent values followed
// by `rot_dim` rotated key values,
//     rows[page][position in page][kv_rank + rot_dim]
// with the same block table as the key/value caches (`block_table[s][i]` = page of positions
// [i * page_tokens, (i + 1) * page_tokens) of the step's s-th sequence).
//
// mu_rotary          rotates `dims` entries (entry i with entry i + dims/2) of each head's slice by
//                    position * freq[i]; cos and sin are scaled by `mag`; entries past `dims` are copied.
//                    Angles, cos and sin in float32.  May write to another buffer of another type.
// mu_latent_append   per token: RMS norm (float32) of the first kv_rank values of the down-projection,
//                    rotation of the last rot_dim, both written to the token's cache row.
// mu_latent_attention  every head's query is [kv_rank + rot_dim] wide (the unrotated part already carried
//                    into latent space by the key up-projection); score = q . row * scale over rows
//                    0..position; softmax; the output is the weighted sum of the rows' first kv_rank values
//                    (the value up-projection follows as a product).  One block per (token, head, split of
//                    the keys), a warp per key, each lane holding its share of the row in registers so that
//                    the row is read once for the score and the sum; float32 throughout; partial results
//                    of splits are merged by a second kernel in split order.
//                    Options for other designs: `pairs` (mu_latent_append: entry 2i turns with entry 2i + 1
//                    instead of entry i with entry i + dims/2) and `sink` (one float per head: the softmax's
//                    denominator also counts exp(sink[h]), unscaled and with no value behind it).
#include "common.cuh"

#include <math.h>

namespace mu {

template <typename TI, typename TO>
__global__ void rotary_kernel(const TI* __restrict__ x, long long ldx, int x_head_stride, TO* __restrict__ y,
                              long long ldy, int y_head_stride, const int* __restrict__ tok_pos,
                              const float* __restrict__ freqs, float mag, int n_heads, int dims, int width) {
    pdl_trigger();
    pdl_wait();
    const int t = blockIdx.x, half = dims / 2;
    const float pos = (float)tok_pos[t];
    const TI* src = x + (long long)t * ldx;
    TO* dst = y + (long long)t * ldy;
    const int per_head = width - half;                 // a thread takes a pair, or one entry past `dims`
    for (int i = threadIdx.x; i < n_heads * per_head; i += blockDim.x) {
        const int h = i / per_head, e = i % per_head;
        const TI* s = src + (long long)h * x_head_stride;
        TO* d = dst + (long long)h * y_head_stride;
        if (e < half) {
            float sn, cs;
            sincosf(pos * freqs[e], &sn, &cs);
            sn *= mag; cs *= mag;
            const float u = to_float(s[e]), v = to_float(s[e + half]);
            d[e] = from_float<TO>(u * cs - v * sn);
            d[e + half] = from_float<TO>(v * cs + u * sn);
        } else {
            d[e + half] = from_float<TO>(to_float(s[e + half]));
        }
    }
}

// With q (and qa): the same block also rotates the token's queries (every head's rot_dim entries at q + h *
// q_head_stride) into qa + h * qa_head_stride as float32, so that a step needs one launch for both.  With dkv
// null only the queries are rotated (a layer that reads another layer's cache).
template <typename T>
__global__ void latent_append_kernel(const T* __restrict__ dkv, long long ld, const float* __restrict__ norm_w, float eps,
                                     const float* __restrict__ freqs, float mag, int rot_dims, int kv_rank, int rot_dim,
                                     const int* __restrict__ tok_pos, const int* __restrict__ tok_seq,
                                     const int* __restrict__ block_table, int max_pages, int page_tokens,
                                     T* __restrict__ rows, const T* __restrict__ q, long long ldq, int q_head_stride,
                                     float* __restrict__ qa, long long ldqa, int qa_head_stride, int n_heads,
                                     int pairs) {
    __shared__ float scratch[32];
    pdl_trigger();
    pdl_wait();
    const int t = blockIdx.x;
    const int p = tok_pos[t];
    if (q) {
        const int half = rot_dims / 2, per_head = rot_dim - half;
        const float pos = (float)p;
        const T* src = q + (long long)t * ldq;
        float* dst = qa + (long long)t * ldqa;
        for (int i = threadIdx.x; i < n_heads * per_head; i += blockDim.x) {
            const int h = i / per_head, e = i % per_head;
            const T* s = src + (long long)h * q_head_stride;
            float* d = dst + (long long)h * qa_head_stride;
            if (e < half) {
                float sn, cs;
                sincosf(pos * freqs[e], &sn, &cs);
                sn *= mag; cs *= mag;
                const int lo = pairs ? 2 * e : e, hi = pairs ? 2 * e + 1 : e + half;
                const float u = to_float(s[lo]), v = to_float(s[hi]);
                d[lo] = u * cs - v * sn;
                d[hi] = v * cs + u * sn;
            } else {
                d[e + half] = to_float(s[e + half]);
            }
        }
    }
    if (!dkv) return;
    const long long page = block_table[(long long)tok_seq[t] * max_pages + p / page_tokens];
    const int width = kv_rank + rot_dim;
    T* dst = rows + (page * page_tokens + p % page_tokens) * width;
    const T* src = dkv + (long long)t * ld;
    float s = 0.0f;
    for (int d = threadIdx.x; d < kv_rank; d += blockDim.x) {
        const float v = to_float(src[d]);
        s += v * v;
    }
    const float inv = 1.0f / sqrtf(block_sum(s, scratch) / (float)kv_rank + eps);
    for (int d = threadIdx.x; d < kv_rank; d += blockDim.x) dst[d] = from_float<T>(to_float(src[d]) * inv * norm_w[d]);
    const int half = rot_dims / 2;
    const float pos = (float)p;
    src += kv_rank;
    dst += kv_rank;
    for (int e = threadIdx.x; e < rot_dim - half; e += blockDim.x) {
        if (e < half) {
            float sn, cs;
            sincosf(pos * freqs[e], &sn, &cs);
            sn *= mag; cs *= mag;
            const int lo = pairs ? 2 * e : e, hi = pairs ? 2 * e + 1 : e + half;
            const float u = to_float(src[lo]), v = to_float(src[hi]);
            dst[lo] = from_float<T>(u * cs - v * sn);
            dst[hi] = from_float<T>(v * cs + u * sn);
        } else {
            dst[e + half] = src[e + half];
        }
    }
}

constexpr int LA_WARPS = 4;

// NPL: row entries per lane (the row is NPL * 32 wide at most).
template <typename T, int NPL>
__global__ void __launch_bounds__(LA_WARPS * 32)
latent_attention_kernel(const float* __restrict__ q, const T* __restrict__ rows, const int* __restrict__ block_table,
                        int max_pages, int page_tokens, const int* __restrict__ tok_pos,
                        const int* __restrict__ tok_seq, int n_heads, int kv_rank, int width, float scale, int n_splits,
                        T* __restrict__ out, long long ldo, float* __restrict__ part_o, float* __restrict__ part_ml,
                        const float* __restrict__ sink) {
    __shared__ float sm_m[LA_WARPS], sm_l[LA_WARPS];
    extern __shared__ float sm_acc[];                  // [LA_WARPS][kv_rank]
    pdl_trigger();
    pdl_wait();
    const int item = blockIdx.x, t = item / n_heads, split = blockIdx.y;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int n_keys = tok_pos[t] + 1;
    // the split's keys: whole groups of LA_WARPS keys, so that a split's warps stay in step
    int per = (n_keys + n_splits - 1) / n_splits;
    per = (per + LA_WARPS - 1) / LA_WARPS * LA_WARPS;
    const int lo = split * per, hi = min(n_keys, lo + per);
    const int* pages = block_table + (long long)tok_seq[t] * max_pages;
    const float* qrow = q + (long long)item * width;
    float qr[NPL], acc[NPL];
#pragma unroll
    for (int i = 0; i < NPL; ++i) {
        const int d = lane + 32 * i;
        qr[i] = d < width ? qrow[d] * scale : 0.0f;
        acc[i] = 0.0f;
    }
    float m = -INFINITY, l = 0.0f;
    for (int j = lo + warp; j < hi; j += LA_WARPS) {
        const T* row = rows + ((long long)pages[j / page_tokens] * page_tokens + j % page_tokens) * width;
        float kr[NPL], s = 0.0f;
#pragma unroll
        for (int i = 0; i < NPL; ++i) {
            const int d = lane + 32 * i;
            kr[i] = d < width ? to_float(row[d]) : 0.0f;
            s += qr[i] * kr[i];
        }
        s = warp_sum(s);
        const float m_new = fmaxf(m, s);
        const float corr = expf(m - m_new), p = expf(s - m_new);     // exp(-inf) = 0 at the first key
        l = l * corr + p;
#pragma unroll
        for (int i = 0; i < NPL; ++i) acc[i] = acc[i] * corr + p * kr[i];
        m = m_new;
    }
    if (lane == 0) { sm_m[warp] = m; sm_l[warp] = l; }
#pragma unroll
    for (int i = 0; i < NPL; ++i) {
        const int d = lane + 32 * i;
        if (d < kv_rank) sm_acc[warp * kv_rank + d] = acc[i];
    }
    __syncthreads();
    float top = -INFINITY;
#pragma unroll
    for (int w = 0; w < LA_WARPS; ++w) top = fmaxf(top, sm_m[w]);
    float f[LA_WARPS], sum = 0.0f;
#pragma unroll
    for (int w = 0; w < LA_WARPS; ++w) {
        f[w] = sm_m[w] == -INFINITY ? 0.0f : expf(sm_m[w] - top);
        sum += sm_l[w] * f[w];
    }
    if (n_splits == 1) {
        T* dst = out + (long long)t * ldo + (long long)(item % n_heads) * kv_rank;
        float inv = 1.0f / sum;
        if (sink) {
            // one more term exp(sink) in the denominator: everything moves to the larger of the two maxima
            const float sk = sink[item % n_heads], top2 = fmaxf(top, sk);
            const float g = expf(top - top2);
            inv = g / (sum * g + expf(sk - top2));
        }
        for (int d = threadIdx.x; d < kv_rank; d += blockDim.x) {
            float v = 0.0f;
#pragma unroll
            for (int w = 0; w < LA_WARPS; ++w) v += sm_acc[w * kv_rank + d] * f[w];
            dst[d] = from_float<T>(v * inv);
        }
        return;
    }
    float* po = part_o + ((long long)item * n_splits + split) * kv_rank;
    for (int d = threadIdx.x; d < kv_rank; d += blockDim.x) {
        float v = 0.0f;
#pragma unroll
        for (int w = 0; w < LA_WARPS; ++w) v += sm_acc[w * kv_rank + d] * f[w];
        po[d] = v;
    }
    if (threadIdx.x == 0) {
        part_ml[((long long)item * n_splits + split) * 2] = top;
        part_ml[((long long)item * n_splits + split) * 2 + 1] = sum;
    }
}

template <typename T>
__global__ void latent_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml, int n_heads,
                                    int kv_rank, int n_splits, T* __restrict__ out, long long ldo,
                                    const float* __restrict__ sink) {
    pdl_trigger();
    pdl_wait();
    __shared__ float factor[64];                       // the parts' weights, 64 parts at a time
    const int item = blockIdx.x, t = item / n_heads;
    const float* ml = part_ml + (long long)item * n_splits * 2;
    float top = sink ? sink[item % n_heads] : -INFINITY;
    for (int s = 0; s < n_splits; ++s) top = fmaxf(top, ml[2 * s]);
    float sum = sink ? expf(sink[item % n_heads] - top) : 0.0f;
    for (int s = 0; s < n_splits; ++s) sum += ml[2 * s] == -INFINITY ? 0.0f : ml[2 * s + 1] * expf(ml[2 * s] - top);
    const float inv = 1.0f / sum;
    T* dst = out + (long long)t * ldo + (long long)(item % n_heads) * kv_rank;
    constexpr int MAX_D = 8;                           // output entries a thread keeps (kv_rank <= 8 * blockDim.x)
    float v[MAX_D] = {};
    for (int s0 = 0; s0 < n_splits; s0 += 64) {
        __syncthreads();
        if (threadIdx.x < 64 && s0 + threadIdx.x < n_splits) {
            const float m = ml[2 * (s0 + threadIdx.x)];
            factor[threadIdx.x] = m == -INFINITY ? 0.0f : expf(m - top);
        }
        __syncthreads();
        const int n = min(64, n_splits - s0);
#pragma unroll
        for (int i = 0; i < MAX_D; ++i) {
            const int d = threadIdx.x + i * blockDim.x;
            if (d < kv_rank)
                for (int s = 0; s < n; ++s)
                    if (factor[s] != 0.0f) v[i] += part_o[((long long)item * n_splits + s0 + s) * kv_rank + d] * factor[s];
        }
    }
#pragma unroll
    for (int i = 0; i < MAX_D; ++i) {
        const int d = threadIdx.x + i * blockDim.x;
        if (d < kv_rank) dst[d] = from_float<T>(v[i] * inv);
    }
}

template <typename T, int NPL>
int launch_latent_attention(const float* q, const T* rows, const int* block_table, int max_pages, int page_tokens,
                            const int* tok_pos, const int* tok_seq, int n_tokens, int n_heads, int kv_rank, int width,
                            float scale, int n_splits, T* out, long long ldo, float* part_o, float* part_ml,
                            const float* sink, cudaStream_t s) {
    const size_t smem = (size_t)LA_WARPS * kv_rank * sizeof(float);
    return launch_pdl(latent_attention_kernel<T, NPL>, dim3(n_tokens * n_heads, n_splits), dim3(LA_WARPS * 32), smem, s, 1,
                      q, rows, block_table, max_pages, page_tokens, tok_pos, tok_seq, n_heads, kv_rank, width, scale,
                      n_splits, out, ldo, part_o, part_ml, sink);
}

template <typename T>
int latent_attention_any(const float* q, const T* rows, const int* block_table, int max_pages, int page_tokens,
                         const int* tok_pos, const int* tok_seq, int n_tokens, int n_heads, int kv_rank, int width,
                         float scale, int n_splits, T* out, long long ldo, float* part_o, float* part_ml,
                         const float* sink, cudaStream_t s) {
#define MU_LA(N)                                                                                                      \
    if (width <= 32 * N)                                                                                              \
        return launch_latent_attention<T, N>(q, rows, block_table, max_pages, page_tokens, tok_pos, tok_seq, n_tokens, \
                                             n_heads, kv_rank, width, scale, n_splits, out, ldo, part_o, part_ml, sink, s);
    MU_LA(2) MU_LA(4) MU_LA(6) MU_LA(8) MU_LA(12) MU_LA(16) MU_LA(20) MU_LA(24) MU_LA(32) MU_LA(48)
#undef MU_LA
    return MU_ERR_UNSUPPORTED_SIZE;
}

}  // namespace mu

MU_EXPORT int mu_rotary(const void* x, long long ldx, int x_head_stride, int x_bf16, void* y, long long ldy,
                        int y_head_stride, int y_bf16, const int* tok_pos, const float* freqs, float mag, int n_tokens,
                        int n_heads, int dims, int width, void* stream) {
    if (n_tokens <= 0 || n_heads <= 0) return MU_OK;
    if (!x || !y || !tok_pos || !freqs || dims < 0 || dims % 2 || width < dims) return MU_ERR_BAD_ARGUMENT;
    cudaStream_t s = (cudaStream_t)stream;
    const dim3 grid(n_tokens), block(128);
    typedef __nv_bfloat16 bf;
#define MU_ROT(TI, TO)                                                                                             \
    return mu::launch_pdl(mu::rotary_kernel<TI, TO>, grid, block, 0, s, 1, (const TI*)x, ldx, x_head_stride, (TO*)y, \
                          ldy, y_head_stride, tok_pos, freqs, mag, n_heads, dims, width)
    if (x_bf16 && y_bf16) MU_ROT(bf, bf);
    if (x_bf16) MU_ROT(bf, float);
    if (y_bf16) MU_ROT(float, bf);
    MU_ROT(float, float);
#undef MU_ROT
}

// dkv may be null (no cache row is written) if q is given; q may be null (no queries are rotated).
MU_EXPORT int mu_latent_append(const void* dkv, long long ld, const float* norm_w, float eps, const float* freqs,
                               float mag, int rot_dims, int kv_rank, int rot_dim, const int* tok_pos,
                               const int* tok_seq, const int* block_table, int max_pages, int page_tokens,
                               int n_tokens, void* rows, int is_bf16, const void* q, long long ldq, int q_head_stride,
                               float* qa, long long ldqa, int qa_head_stride, int n_heads, void* stream, int pairs) {
    if (n_tokens <= 0) return MU_OK;
    if ((!dkv && !q) || !freqs || !tok_pos || kv_rank <= 0 || rot_dim < 0 || rot_dims % 2 || rot_dims > rot_dim ||
        (dkv && (!norm_w || !tok_seq || !block_table || !rows || page_tokens <= 0)) || (q && (!qa || n_heads <= 0)))
        return MU_ERR_BAD_ARGUMENT;
    cudaStream_t s = (cudaStream_t)stream;
    const dim3 grid(n_tokens), block(kv_rank >= 512 ? 256 : 128);
    if (is_bf16)
        return mu::launch_pdl(mu::latent_append_kernel<__nv_bfloat16>, grid, block, 0, s, 1, (const __nv_bfloat16*)dkv,
                              ld, norm_w, eps, freqs, mag, rot_dims, kv_rank, rot_dim, tok_pos, tok_seq, block_table,
                              max_pages, page_tokens, (__nv_bfloat16*)rows, (const __nv_bfloat16*)q, ldq, q_head_stride,
                              qa, ldqa, qa_head_stride, n_heads, pairs);
    return mu::launch_pdl(mu::latent_append_kernel<float>, grid, block, 0, s, 1, (const float*)dkv, ld, norm_w, eps,
                          freqs, mag, rot_dims, kv_rank, rot_dim, tok_pos, tok_seq, block_table, max_pages, page_tokens,
                          (float*)rows, (const float*)q, ldq, q_head_stride, qa, ldqa, qa_head_stride, n_heads, pairs);
}

// q: float32 [n_tokens, n_heads, width]; out: [n_tokens, ldo] with head h at columns h * kv_rank.
// n_splits > 1 needs part_o (n_tokens * n_heads * n_splits * kv_rank floats) and part_ml (... * 2).
MU_EXPORT int mu_latent_attention(const float* q, const void* rows, const int* block_table, int max_pages,
                                  int page_tokens, const int* tok_pos, const int* tok_seq, int n_tokens, int n_heads,
                                  int kv_rank, int width, float scale, int n_splits, void* out, long long ldo,
                                  float* part_o, float* part_ml, int is_bf16, void* stream, const float* sink) {
    if (n_tokens <= 0) return MU_OK;
    if (!q || !rows || !block_table || !tok_pos || !tok_seq || !out || n_heads <= 0 || kv_rank <= 0 || width < kv_rank ||
        n_splits < 1 || n_splits > 65535 || (n_splits > 1 && (!part_o || !part_ml)))
        return MU_ERR_BAD_ARGUMENT;
    if ((size_t)mu::LA_WARPS * kv_rank * sizeof(float) > 48 * 1024) return MU_ERR_UNSUPPORTED_SIZE;
    cudaStream_t s = (cudaStream_t)stream;
    int code;
    if (is_bf16)
        code = mu::latent_attention_any<__nv_bfloat16>(q, (const __nv_bfloat16*)rows, block_table, max_pages, page_tokens,
                                                       tok_pos, tok_seq, n_tokens, n_heads, kv_rank, width, scale,
                                                       n_splits, (__nv_bfloat16*)out, ldo, part_o, part_ml,
                                                       n_splits == 1 ? sink : nullptr, s);
    else
        code = mu::latent_attention_any<float>(q, (const float*)rows, block_table, max_pages, page_tokens, tok_pos,
                                               tok_seq, n_tokens, n_heads, kv_rank, width, scale, n_splits, (float*)out,
                                               ldo, part_o, part_ml, n_splits == 1 ? sink : nullptr, s);
    if (code != MU_OK || n_splits == 1) return code;
    const dim3 grid(n_tokens * n_heads), block(kv_rank > 1024 ? 512 : 128);    // a thread keeps up to 8 entries
    if (is_bf16)
        return mu::launch_pdl(mu::latent_merge_kernel<__nv_bfloat16>, grid, block, 0, s, 1, (const float*)part_o,
                              (const float*)part_ml, n_heads, kv_rank, n_splits, (__nv_bfloat16*)out, ldo, sink);
    return mu::launch_pdl(mu::latent_merge_kernel<float>, grid, block, 0, s, 1, (const float*)part_o,
                          (const float*)part_ml, n_heads, kv_rank, n_splits, (float*)out, ldo, sink);
}

// Merges the partial results of n_splits parts of every (token, head) into out (bfloat16 or float32).
MU_EXPORT int mu_latent_merge(const float* part_o, const float* part_ml, int n_tokens, int n_heads, int kv_rank,
                              int n_splits, void* out, long long ldo, int is_bf16, void* stream, const float* sink) {
    if (n_tokens <= 0) return MU_OK;
    if (!part_o || !part_ml || !out || n_heads <= 0 || kv_rank <= 0 || n_splits < 1) return MU_ERR_BAD_ARGUMENT;
    cudaStream_t s = (cudaStream_t)stream;
    const dim3 grid(n_tokens * n_heads), block(kv_rank > 1024 ? 512 : 128);    // a thread keeps up to 8 entries
    if (is_bf16)
        return mu::launch_pdl(mu::latent_merge_kernel<__nv_bfloat16>, grid, block, 0, s, 1, part_o, part_ml, n_heads,
                              kv_rank, n_splits, (__nv_bfloat16*)out, ldo, sink);
    return mu::launch_pdl(mu::latent_merge_kernel<float>, grid, block, 0, s, 1, part_o, part_ml, n_heads, kv_rank,
                          n_splits, (float*)out, ldo, sink);
}
