// Attention whose heads have one or two score maps, normed and rotated queries and keys, and values of
// their own size, over a paged cache that keeps ONE row per position:
//     row = [ keys: kv head 0 {map 0 | map 1}, kv head 1 {...}, ... | values: kv head 0, kv head 1, ... ]
// (`maps` * dim entries per kv head of keys, vdim entries per kv head of values).  Pages hold `page_tokens`
// rows; block_table[s][i] is the page with positions [i * page_tokens, (i + 1) * page_tokens) of the step's
// s-th sequence.
//
// mu_qk_prepare        per token: every (head, map) slice of the queries and of the keys is brought to unit
//                      rms over its dim entries (eps inside the root), multiplied by a weight shared by all
//                      heads and maps, and its first rot_dims entries are rotated (entry i with entry
//                      i + rot_dims / 2 by the angle position * freq[i]; cos and sin times a magnitude);
//                      queries are written back in place, keys and values go to the token's cache row.
//                      Statistics, angles, cos and sin are float32 whatever the storage type.
//                      Options for other designs: a null weight leaves the slices as they are (no norm);
//                      `pairs` rotates entry 2i with entry 2i + 1 instead of entry i with entry i + rot_dims / 2.
// mu_mapped_attention  per (token, head): softmax attention of each map over the keys the token sees
//                      (positions max(0, p - window + 1) .. p; window 0: all of 0 .. p), both maps over the
//                      same values.  With two maps the result is a1 - lambda * a2, brought to unit rms over
//                      the head's vdim entries and multiplied by out_scale.  Scores, softmax and sums are
//                      float32.  Which warp takes which keys depends on the token's position only, so a
//                      token's result does not depend on the step it ran in.
//                      Options for other designs: `head_scale` (one float per head that multiplies the head's
//                      scores besides `scale`), `sink` (the softmax's denominator counts one more key whose score
//                      is zero and which has no value), `gate` ([T, heads] in the storage type: the head's result
//                      is multiplied by sigmoid(gate[t][h]), computed in float32), `chunk` (c > 0: a token at
//                      position p sees the positions p - p % c .. p only, chunks counted from position 0 of the
//                      sequence; it replaces the window).
#include "common.cuh"

#include <math.h>

namespace mu {

constexpr int MA_WARPS = 4;
constexpr int MA_VPL = 8;          // value entries per lane: vdim <= 256

template <typename TE>
__global__ void __launch_bounds__(128)
qk_prepare_kernel(TE* __restrict__ q, long long ldq, const TE* __restrict__ k, long long ldk,
                  const TE* __restrict__ v, long long ldv, const float* __restrict__ q_weight,
                  const float* __restrict__ k_weight, const float* __restrict__ freqs, float magnitude,
                  int rot_dims, float eps, int n_heads, int n_kv_heads, int maps, int dim, int vdim,
                  const int* __restrict__ tok_pos, const int* __restrict__ tok_seq,
                  const int* __restrict__ block_table, int max_pages, int page_tokens, TE* __restrict__ rows,
                  int pairs) {
    extern __shared__ float staged[];                       // [warps][dim] | cos [rot_dims / 2] | sin [rot_dims / 2]
    pdl_trigger();
    pdl_wait();
    const int t = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
    const int pos = tok_pos[t];
    const int half = rot_dims / 2;
    float* cs_tab = staged + warps * dim;
    float* sn_tab = cs_tab + half;
    // the token's angles once for all its slices
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
        float sn, cs;
        sincosf((float)pos * freqs[i], &sn, &cs);
        cs_tab[i] = cs * magnitude;
        sn_tab[i] = sn * magnitude;
    }
    __syncthreads();
    const int n_q = n_heads * maps, n_k = k ? n_kv_heads * maps : 0;
    const long long width = (long long)n_kv_heads * (maps * dim + vdim);
    TE* row = nullptr;
    if (k) {
        const long long page = block_table[(long long)tok_seq[t] * max_pages + pos / page_tokens];
        row = rows + (page * page_tokens + pos % page_tokens) * width;
    }
    float* mine = staged + warp * dim;
    // blockIdx.y-th share of the token's slices, a warp a slice
    for (int item = blockIdx.y * warps + warp; item < n_q + n_k; item += gridDim.y * warps) {
        const bool is_q = item < n_q;
        const int slice = is_q ? item : item - n_q;
        const TE* src = is_q ? q + (long long)t * ldq + (long long)slice * dim : k + (long long)t * ldk + (long long)slice * dim;
        TE* dst = is_q ? q + (long long)t * ldq + (long long)slice * dim : row + (long long)slice * dim;
        const float* weight = is_q ? q_weight : k_weight;
        float ss = 0.0f;
        for (int d = lane; d < dim; d += 32) {
            const float x = to_float(src[d]);
            mine[d] = x;
            ss += x * x;
        }
        ss = warp_sum(ss);
        const float inv = weight ? 1.0f / sqrtf(ss / (float)dim + eps) : 1.0f;
        __syncwarp();
        for (int d = lane; d < dim; d += 32) {
            float y;
            if (d < rot_dims) {
                // the entry's partner and which of the two it is: (i, i + half) or (2i, 2i + 1)
                const int i = pairs ? d >> 1 : (d < half ? d : d - half);
                const int lo = pairs ? 2 * i : i, hi = pairs ? 2 * i + 1 : i + half;
                const float a = mine[lo] * inv * (weight ? weight[lo] : 1.0f), b = mine[hi] * inv * (weight ? weight[hi] : 1.0f);
                const float cs = cs_tab[i], sn = sn_tab[i];
                y = d == lo ? a * cs - b * sn : b * cs + a * sn;
            } else {
                y = mine[d] * inv * (weight ? weight[d] : 1.0f);
            }
            dst[d] = from_float<TE>(y);
        }
        __syncwarp();
    }
    if (v && blockIdx.y == 0) {
        TE* vdst = row + (long long)n_kv_heads * maps * dim;
        const TE* vsrc = v + (long long)t * ldv;
        for (int d = threadIdx.x; d < n_kv_heads * vdim; d += blockDim.x) vdst[d] = vsrc[d];
    }
}

template <typename TE>
__device__ __forceinline__ float dot_key(const float* qs, const TE* key, int dim, bool vec);

template <>
__device__ __forceinline__ float dot_key<float>(const float* qs, const float* key, int dim, bool vec) {
    float s = 0.0f;
    if (vec) {
        for (int d = 0; d < dim; d += 4) {
            const float4 kk = *reinterpret_cast<const float4*>(key + d);
            s = fmaf(qs[d], kk.x, s);
            s = fmaf(qs[d + 1], kk.y, s);
            s = fmaf(qs[d + 2], kk.z, s);
            s = fmaf(qs[d + 3], kk.w, s);
        }
    } else {
        for (int d = 0; d < dim; ++d) s = fmaf(qs[d], key[d], s);
    }
    return s;
}

template <>
__device__ __forceinline__ float dot_key<__nv_bfloat16>(const float* qs, const __nv_bfloat16* key, int dim, bool vec) {
    float s = 0.0f;
    if (vec) {
        for (int d = 0; d < dim; d += 8) {
            const uint4 raw = *reinterpret_cast<const uint4*>(key + d);
            const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float2 f = __bfloat1622float2(p[i]);
                s = fmaf(qs[d + 2 * i], f.x, s);
                s = fmaf(qs[d + 2 * i + 1], f.y, s);
            }
        }
    } else {
        for (int d = 0; d < dim; ++d) s = fmaf(qs[d], __bfloat162float(key[d]), s);
    }
    return s;
}

// One block per (token, head).  A warp takes every MA_WARPS-th run of 32 keys, counted from the first key the
// token sees: a lane computes the scores of one key (both maps), the warp keeps a running maximum and sum per
// map, and the lanes share the value entries for the weighted sums.  The warps' parts meet in shared memory.
template <typename TE, int MAPS>
__global__ void __launch_bounds__(MA_WARPS * 32)
mapped_attention_kernel(const TE* __restrict__ q, long long ldq, const TE* __restrict__ rows,
                        const int* __restrict__ block_table, int max_pages, int page_tokens,
                        const int* __restrict__ tok_pos, const int* __restrict__ tok_seq, int n_heads,
                        int n_kv_heads, int dim, int vdim, float scale, int window, float lambda, float out_scale,
                        float eps, int unit_rms, int vec, TE* __restrict__ out, long long ldo,
                        const float* __restrict__ head_scale, int sink, const TE* __restrict__ gate, long long ldg,
                        int chunk) {
    extern __shared__ float smem[];
    float* qs = smem;                                        // [MAPS][dim]
    float* part_acc = qs + MAPS * dim;                       // [warps][MAPS][vdim]
    float* part_ml = part_acc + MA_WARPS * MAPS * vdim;      // [warps][MAPS][2]
    __shared__ float scratch[32];
    pdl_trigger();
    pdl_wait();
    const int t = blockIdx.x, h = blockIdx.y, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = h / (n_heads / n_kv_heads);
    const int pos = tok_pos[t];
    if (head_scale) scale *= head_scale[h];
    const int* pages = block_table + (long long)tok_seq[t] * max_pages;
    const long long width = (long long)n_kv_heads * (MAPS * dim + vdim);
    const long long key_off = (long long)g * MAPS * dim, val_off = (long long)n_kv_heads * MAPS * dim + (long long)g * vdim;
    for (int d = threadIdx.x; d < MAPS * dim; d += blockDim.x)
        qs[d] = to_float(q[(long long)t * ldq + (long long)h * MAPS * dim + d]);
    __syncthreads();
    const int first = chunk > 0 ? pos - pos % chunk : window > 0 ? max(0, pos - window + 1) : 0;
    float m_run[MAPS], l_run[MAPS], acc[MAPS][MA_VPL];
#pragma unroll
    for (int a = 0; a < MAPS; ++a) {
        m_run[a] = -INFINITY;
        l_run[a] = 0.0f;
#pragma unroll
        for (int i = 0; i < MA_VPL; ++i) acc[a][i] = 0.0f;
    }
    for (int base = first + warp * 32; base <= pos; base += MA_WARPS * 32) {
        const int j = base + lane;
        const bool live = j <= pos;
        const TE* row = nullptr;
        float s[MAPS];
#pragma unroll
        for (int a = 0; a < MAPS; ++a) s[a] = -INFINITY;
        if (live) {
            row = rows + ((long long)pages[j / page_tokens] * page_tokens + j % page_tokens) * width;
#pragma unroll
            for (int a = 0; a < MAPS; ++a) s[a] = dot_key<TE>(qs + a * dim, row + key_off + a * dim, dim, vec != 0) * scale;
        }
        float p[MAPS];
#pragma unroll
        for (int a = 0; a < MAPS; ++a) {
            const float m_new = fmaxf(m_run[a], warp_max(s[a]));
            const float corr = expf(m_run[a] - m_new);       // 0 at the first run (m_run is -inf, m_new finite)
            p[a] = live ? expf(s[a] - m_new) : 0.0f;
            l_run[a] = l_run[a] * corr + warp_sum(p[a]);
            m_run[a] = m_new;
#pragma unroll
            for (int i = 0; i < MA_VPL; ++i) acc[a][i] *= corr;
        }
        const int n_live = min(32, pos - base + 1);
        const unsigned long long mine = (unsigned long long)(uintptr_t)row;
        for (int jj = 0; jj < n_live; ++jj) {
            const TE* vrow = reinterpret_cast<const TE*>((uintptr_t)__shfl_sync(0xffffffffu, mine, jj)) + val_off;
            float pj[MAPS];
#pragma unroll
            for (int a = 0; a < MAPS; ++a) pj[a] = __shfl_sync(0xffffffffu, p[a], jj);
#pragma unroll
            for (int i = 0; i < MA_VPL; ++i) {
                const int d = lane + 32 * i;
                if (d < vdim) {
                    const float x = to_float(vrow[d]);
#pragma unroll
                    for (int a = 0; a < MAPS; ++a) acc[a][i] = fmaf(pj[a], x, acc[a][i]);
                }
            }
        }
    }
#pragma unroll
    for (int a = 0; a < MAPS; ++a) {
        if (lane == 0) {
            part_ml[(warp * MAPS + a) * 2] = m_run[a];
            part_ml[(warp * MAPS + a) * 2 + 1] = l_run[a];
        }
#pragma unroll
        for (int i = 0; i < MA_VPL; ++i) {
            const int d = lane + 32 * i;
            if (d < vdim) part_acc[(warp * MAPS + a) * vdim + d] = acc[a][i];
        }
    }
    __syncthreads();
    // the warps' parts in warp order; then the maps' difference and the head's unit rms
    float sq = 0.0f;
    for (int d = threadIdx.x; d < vdim; d += blockDim.x) {
        float o[MAPS];
#pragma unroll
        for (int a = 0; a < MAPS; ++a) {
            float top = sink ? 0.0f : -INFINITY;
            for (int w = 0; w < MA_WARPS; ++w) top = fmaxf(top, part_ml[(w * MAPS + a) * 2]);
            float num = 0.0f, den = sink ? expf(-top) : 0.0f;
            for (int w = 0; w < MA_WARPS; ++w) {
                const float mw = part_ml[(w * MAPS + a) * 2];
                const float f = mw == -INFINITY ? 0.0f : expf(mw - top);
                num += part_acc[(w * MAPS + a) * vdim + d] * f;
                den += part_ml[(w * MAPS + a) * 2 + 1] * f;
            }
            o[a] = num / den;
        }
        const float r = MAPS == 2 ? o[0] - lambda * o[MAPS - 1] : o[0];
        part_acc[d] = r;          // (warp 0, map 0)'s place: each entry is read and written by this thread only
        sq += r * r;
    }
    float mult = out_scale;
    if (unit_rms) mult *= 1.0f / sqrtf(block_sum(sq, scratch) / (float)vdim + eps);
    if (gate) mult *= 1.0f / (1.0f + expf(-to_float(gate[(long long)t * ldg + h])));
    __syncthreads();
    for (int d = threadIdx.x; d < vdim; d += blockDim.x)
        out[(long long)t * ldo + (long long)h * vdim + d] = from_float<TE>(part_acc[d] * mult);
}

// Single-token steps.  A block takes one (token, kv head) and every MD_SPLITS-th page of what the token sees
// (page index modulo MD_SPLITS = blockIdx.z, so the share does not depend on the batch): the page's keys and values
// of that kv head are staged in shared memory once and serve all query heads of the group, a warp a head, a lane a
// key for the scores and a lane a value entry for the sums.  Each (token, head, map, share) leaves a maximum, a sum
// and unnormalised values; mapped_merge_kernel puts the shares together in their order and finishes the head.
constexpr int MD_SPLITS = 16;
constexpr int MD_KEYS = 64;         // keys staged at a time: one page

template <typename TE, int MAPS>
__global__ void __launch_bounds__(128)
mapped_decode_kernel(const TE* __restrict__ q, long long ldq, const TE* __restrict__ rows,
                     const int* __restrict__ block_table, int max_pages, const int* __restrict__ tok_pos,
                     const int* __restrict__ tok_seq, int n_heads, int n_kv_heads, int dim, int vdim, float scale,
                     int window, int vec, float* __restrict__ part_acc, float* __restrict__ part_ml,
                     const float* __restrict__ head_scale, int chunk) {
    extern __shared__ __align__(16) unsigned char md_raw[];
    const int kw = MAPS * dim, rw = kw + vdim;                 // the kv head's entries of a row
    const int pitch = rw + (vec ? 16 / (int)sizeof(TE) : 1);   // rows start in different banks
    TE* tile = reinterpret_cast<TE*>(md_raw);                  // [MD_KEYS][pitch]: keys (both maps), then values
    float* qs = reinterpret_cast<float*>(md_raw + (((size_t)MD_KEYS * pitch * sizeof(TE) + 15) / 16) * 16);   // [group][kw]
    pdl_trigger();
    pdl_wait();
    const int t = blockIdx.x, g = blockIdx.y, share = blockIdx.z;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, warps = blockDim.x >> 5;
    const int group = n_heads / n_kv_heads;
    const int pos = tok_pos[t];
    const int first = chunk > 0 ? pos - pos % chunk : window > 0 ? max(0, pos - window + 1) : 0;
    const int page_lo = first / MD_KEYS, page_hi = pos / MD_KEYS;
    const int* pages = block_table + (long long)tok_seq[t] * max_pages;
    const long long width = (long long)n_kv_heads * rw;
    const long long key_off = (long long)g * kw, val_off = (long long)n_kv_heads * kw + (long long)g * vdim;
    for (int i = tid; i < group * kw; i += blockDim.x)
        qs[i] = to_float(q[(long long)t * ldq + (long long)g * group * kw + i]);
    // heads of the group this warp takes: warp, warp + warps, ... (at most MD_HEADS of them)
    constexpr int MD_HEADS = 4;
    float m_run[MD_HEADS][MAPS], l_run[MD_HEADS][MAPS], acc[MD_HEADS][MAPS][MA_VPL];
#pragma unroll
    for (int u = 0; u < MD_HEADS; ++u)
#pragma unroll
        for (int a = 0; a < MAPS; ++a) {
            m_run[u][a] = -INFINITY;
            l_run[u][a] = 0.0f;
#pragma unroll
            for (int i = 0; i < MA_VPL; ++i) acc[u][a][i] = 0.0f;
        }
    int pg = page_lo + ((share - page_lo) % MD_SPLITS + MD_SPLITS) % MD_SPLITS;     // the first page >= page_lo of this share
    for (; pg <= page_hi; pg += MD_SPLITS) {
        __syncthreads();                                       // the page before is done with (and qs is written)
        const TE* src = rows + (long long)pages[pg] * MD_KEYS * width;
        if (vec) {
            constexpr int E = 16 / (int)sizeof(TE);
            const int kc = kw / E, vc = vdim / E;
            for (int i = tid; i < MD_KEYS * (kc + vc); i += blockDim.x) {
                const int r = i / (kc + vc), c = i % (kc + vc);
                const TE* from = c < kc ? src + r * width + key_off + c * E : src + r * width + val_off + (c - kc) * E;
                *reinterpret_cast<uint4*>(tile + r * pitch + c * E) = *reinterpret_cast<const uint4*>(from);
            }
        } else {
            for (int i = tid; i < MD_KEYS * rw; i += blockDim.x) {
                const int r = i / rw, c = i % rw;
                tile[r * pitch + c] = c < kw ? src[r * width + key_off + c] : src[r * width + val_off + (c - kw)];
            }
        }
        __syncthreads();
        const int key0 = pg * MD_KEYS;
#pragma unroll
        for (int u = 0; u < MD_HEADS; ++u) {
            const int hg = warp + u * warps;                   // the head's place in its group
            if (hg >= group) break;
            const float scale_h = head_scale ? scale * head_scale[g * group + hg] : scale;
#pragma unroll
            for (int half = 0; half < MD_KEYS / 32; ++half) {
                const int jl = half * 32 + lane, j = key0 + jl;
                const bool live = j >= first && j <= pos;
                if (__ballot_sync(0xffffffffu, live) == 0u) continue;
                float p[MAPS];
#pragma unroll
                for (int a = 0; a < MAPS; ++a) {
                    const float sc = live ? dot_key<TE>(qs + hg * kw + a * dim, tile + jl * pitch + a * dim, dim, vec != 0) * scale_h
                                          : -INFINITY;
                    const float m_new = fmaxf(m_run[u][a], warp_max(sc));
                    const float corr = expf(m_run[u][a] - m_new);
                    p[a] = live ? expf(sc - m_new) : 0.0f;
                    l_run[u][a] = l_run[u][a] * corr + warp_sum(p[a]);
                    m_run[u][a] = m_new;
#pragma unroll
                    for (int i = 0; i < MA_VPL; ++i) acc[u][a][i] *= corr;
                }
                for (int jj = 0; jj < 32; ++jj) {
                    float pj[MAPS];
#pragma unroll
                    for (int a = 0; a < MAPS; ++a) pj[a] = __shfl_sync(0xffffffffu, p[a], jj);
                    const TE* vrow = tile + (half * 32 + jj) * pitch + kw;
#pragma unroll
                    for (int i = 0; i < MA_VPL; ++i) {
                        const int d = lane + 32 * i;
                        if (d < vdim) {
                            const float x = to_float(vrow[d]);
#pragma unroll
                            for (int a = 0; a < MAPS; ++a) acc[u][a][i] = fmaf(pj[a], x, acc[u][a][i]);
                        }
                    }
                }
            }
        }
    }
#pragma unroll
    for (int u = 0; u < MD_HEADS; ++u) {
        const int hg = warp + u * warps;
        if (hg >= group) break;
        const int h = g * group + hg;
#pragma unroll
        for (int a = 0; a < MAPS; ++a) {
            const long long item = (((long long)t * n_heads + h) * MAPS + a) * MD_SPLITS + share;
            if (lane == 0) {
                part_ml[item * 2] = m_run[u][a];
                part_ml[item * 2 + 1] = l_run[u][a];
            }
#pragma unroll
            for (int i = 0; i < MA_VPL; ++i) {
                const int d = lane + 32 * i;
                if (d < vdim) part_acc[item * vdim + d] = acc[u][a][i];
            }
        }
    }
}

template <typename TE, int MAPS>
__global__ void __launch_bounds__(128)
mapped_merge_kernel(const float* __restrict__ part_acc, const float* __restrict__ part_ml, int n_heads, int vdim,
                    float lambda, float out_scale, float eps, int unit_rms, TE* __restrict__ out, long long ldo,
                    int sink, const TE* __restrict__ gate, long long ldg) {
    extern __shared__ float merged[];                        // [vdim]
    __shared__ float scratch[32];
    __shared__ float factor[MAPS][MD_SPLITS];
    pdl_trigger();
    pdl_wait();
    const int t = blockIdx.x, h = blockIdx.y;
    const long long item0 = ((long long)t * n_heads + h) * MAPS * MD_SPLITS;
    if (threadIdx.x < MAPS) {
        const int a = threadIdx.x;
        float top = sink ? 0.0f : -INFINITY, den = 0.0f;
        for (int s = 0; s < MD_SPLITS; ++s) top = fmaxf(top, part_ml[(item0 + a * MD_SPLITS + s) * 2]);
        if (sink) den = expf(-top);
        for (int s = 0; s < MD_SPLITS; ++s) {
            const float m = part_ml[(item0 + a * MD_SPLITS + s) * 2];
            const float f = m == -INFINITY ? 0.0f : expf(m - top);
            factor[a][s] = f;
            den += part_ml[(item0 + a * MD_SPLITS + s) * 2 + 1] * f;
        }
        for (int s = 0; s < MD_SPLITS; ++s) factor[a][s] /= den;
    }
    __syncthreads();
    float sq = 0.0f;
    for (int d = threadIdx.x; d < vdim; d += blockDim.x) {
        float o[MAPS];
#pragma unroll
        for (int a = 0; a < MAPS; ++a) {
            float num = 0.0f;
            for (int s = 0; s < MD_SPLITS; ++s)
                if (factor[a][s] != 0.0f) num += part_acc[(item0 + a * MD_SPLITS + s) * vdim + d] * factor[a][s];
            o[a] = num;
        }
        const float r = MAPS == 2 ? o[0] - lambda * o[MAPS - 1] : o[0];
        merged[d] = r;
        sq += r * r;
    }
    float mult = out_scale;
    if (unit_rms) mult *= 1.0f / sqrtf(block_sum(sq, scratch) / (float)vdim + eps);
    if (gate) mult *= 1.0f / (1.0f + expf(-to_float(gate[(long long)t * ldg + h])));
    __syncthreads();
    for (int d = threadIdx.x; d < vdim; d += blockDim.x)
        out[(long long)t * ldo + (long long)h * vdim + d] = from_float<TE>(merged[d] * mult);
}

}  // namespace mu

// q [T, n_heads * maps * dim] is normed and rotated in place; k [T, n_kv_heads * maps * dim] and
// v [T, n_kv_heads * vdim] (both may be null: a layer that reads another layer's rows) go to the cache rows.
MU_EXPORT int mu_qk_prepare(void* q, long long ldq, const void* k, long long ldk, const void* v, long long ldv,
                            const float* q_weight, const float* k_weight, const float* freqs, float magnitude,
                            int rot_dims, float eps, int n_tokens, int n_heads, int n_kv_heads, int maps, int dim,
                            int vdim, const int* tok_pos, const int* tok_seq, const int* block_table, int max_pages,
                            int page_tokens, void* rows, int is_bf16, void* stream, int pairs) {
    if (n_tokens <= 0) return MU_OK;
    if (!q || !tok_pos || dim <= 0 || maps < 1 || maps > 2 || rot_dims < 0 || rot_dims % 2 ||
        rot_dims > dim || (rot_dims > 0 && !freqs) || (k != nullptr) != (v != nullptr))
        return MU_ERR_BAD_ARGUMENT;
    if (k && ((k_weight != nullptr) != (q_weight != nullptr) || !tok_seq || !block_table || !rows || page_tokens <= 0))
        return MU_ERR_BAD_ARGUMENT;
    if (dim > 4096) return MU_ERR_UNSUPPORTED_SIZE;
    cudaStream_t s = (cudaStream_t)stream;
    const int threads = 128;
    const size_t smem = ((size_t)(threads / 32) * dim + rot_dims) * sizeof(float);
    // a token's slices are spread over several blocks, a warp a slice
    const int items = (n_heads + (k ? n_kv_heads : 0)) * maps;
    const int shares = (items + 3) / 4;
    const dim3 grid(n_tokens, shares);
    typedef __nv_bfloat16 bf;
    if (is_bf16)
        return mu::launch_pdl(mu::qk_prepare_kernel<bf>, grid, dim3(threads), smem, s, 1, (bf*)q, ldq,
                              (const bf*)k, ldk, (const bf*)v, ldv, q_weight, k_weight, freqs, magnitude, rot_dims, eps,
                              n_heads, n_kv_heads, maps, dim, vdim, tok_pos, tok_seq, block_table, max_pages,
                              page_tokens, (bf*)rows, pairs);
    return mu::launch_pdl(mu::qk_prepare_kernel<float>, grid, dim3(threads), smem, s, 1, (float*)q, ldq,
                          (const float*)k, ldk, (const float*)v, ldv, q_weight, k_weight, freqs, magnitude, rot_dims,
                          eps, n_heads, n_kv_heads, maps, dim, vdim, tok_pos, tok_seq, block_table, max_pages,
                          page_tokens, (float*)rows, pairs);
}

MU_EXPORT int mu_mapped_attention(const void* q, long long ldq, const void* rows, const int* block_table,
                                  int max_pages, int page_tokens, const int* tok_pos, const int* tok_seq,
                                  int n_tokens, int n_heads, int n_kv_heads, int maps, int dim, int vdim, float scale,
                                  int window, float lambda, float out_scale, float eps, int unit_rms, void* out,
                                  long long ldo, int is_bf16, void* stream, const float* head_scale, int sink,
                                  const void* gate, long long ldg, int chunk) {
    if (n_tokens <= 0) return MU_OK;
    if (!q || !rows || !block_table || !tok_pos || !tok_seq || !out || n_heads <= 0 || n_kv_heads <= 0 ||
        n_heads % n_kv_heads || maps < 1 || maps > 2 || dim <= 0 || vdim <= 0 || page_tokens <= 0 || window < 0 ||
        chunk < 0)
        return MU_ERR_BAD_ARGUMENT;
    if (vdim > 32 * mu::MA_VPL) return MU_ERR_UNSUPPORTED_SIZE;
    const size_t smem = ((size_t)maps * dim + (size_t)mu::MA_WARPS * maps * (vdim + 2)) * sizeof(float);
    if (smem > 48 * 1024) return MU_ERR_UNSUPPORTED_SIZE;
    // 16-byte pieces of a key: every slice of a row must start on such a boundary
    const int per = is_bf16 ? 8 : 4;
    const int vec = dim % per == 0 && (n_kv_heads * vdim) % per == 0 && ((uintptr_t)rows & 15) == 0;
    cudaStream_t s = (cudaStream_t)stream;
    const dim3 grid(n_tokens, n_heads), block(mu::MA_WARPS * 32);
    typedef __nv_bfloat16 bf;
#define MU_MAPPED(TE, M)                                                                                              \
    return mu::launch_pdl(mu::mapped_attention_kernel<TE, M>, grid, block, smem, s, 1, (const TE*)q, ldq,             \
                          (const TE*)rows, block_table, max_pages, page_tokens, tok_pos, tok_seq, n_heads, n_kv_heads, \
                          dim, vdim, scale, window, lambda, out_scale, eps, unit_rms, vec, (TE*)out, ldo, head_scale,  \
                          sink, (const TE*)gate, ldg, chunk)
    if (is_bf16) {
        if (maps == 2) MU_MAPPED(bf, 2);
        MU_MAPPED(bf, 1);
    }
    if (maps == 2) MU_MAPPED(float, 2);
    MU_MAPPED(float, 1);
#undef MU_MAPPED
}

// Whether mu_mapped_attention_decode takes these sizes (a staged page and the group's queries fit shared memory).
MU_EXPORT int mu_mapped_decode_fits(int n_heads, int n_kv_heads, int maps, int dim, int vdim, int page_tokens, int is_bf16) {
    if (n_kv_heads <= 0 || n_heads % n_kv_heads || page_tokens != mu::MD_KEYS || vdim > 32 * mu::MA_VPL) return 0;
    const int group = n_heads / n_kv_heads, esize = is_bf16 ? 2 : 4;
    const size_t smem = (size_t)mu::MD_KEYS * (maps * dim + vdim + 16 / esize) * esize + 16 + (size_t)group * maps * dim * sizeof(float);
    return group <= 16 && smem <= 160 * 1024;
}

// Floats of scratch a single-token step needs: part_acc, and after it part_ml.
MU_EXPORT long long mu_mapped_decode_scratch(int n_tokens, int n_heads, int maps, int vdim) {
    return (long long)n_tokens * n_heads * maps * mu::MD_SPLITS * (vdim + 2);
}

// The same attention for steps in which every token is the one token of its sequence: pages shared out over
// blocks, the query heads of a kv head together; `scratch` holds mu_mapped_decode_scratch floats.  Page of 64.
MU_EXPORT int mu_mapped_attention_decode(const void* q, long long ldq, const void* rows, const int* block_table,
                                         int max_pages, int page_tokens, const int* tok_pos, const int* tok_seq,
                                         int n_tokens, int n_heads, int n_kv_heads, int maps, int dim, int vdim,
                                         float scale, int window, float lambda, float out_scale, float eps, int unit_rms,
                                         float* scratch, void* out, long long ldo, int is_bf16, void* stream,
                                         const float* head_scale, int sink, const void* gate, long long ldg, int chunk) {
    if (n_tokens <= 0) return MU_OK;
    if (!q || !rows || !block_table || !tok_pos || !tok_seq || !out || !scratch || n_heads <= 0 || n_kv_heads <= 0 ||
        n_heads % n_kv_heads || maps < 1 || maps > 2 || dim <= 0 || vdim <= 0 || window < 0 || chunk < 0)
        return MU_ERR_BAD_ARGUMENT;
    const int group = n_heads / n_kv_heads;
    if (page_tokens != mu::MD_KEYS || vdim > 32 * mu::MA_VPL || group > 16) return MU_ERR_UNSUPPORTED_SIZE;
    const int esize = is_bf16 ? 2 : 4, per = 16 / esize;
    const int vec = dim % per == 0 && vdim % per == 0 && ((uintptr_t)rows & 15) == 0;
    const int rw = maps * dim + vdim, pitch = rw + (vec ? per : 1);
    const size_t smem = (((size_t)mu::MD_KEYS * pitch * esize + 15) / 16) * 16 + (size_t)group * maps * dim * sizeof(float);
    if (smem > 200 * 1024) return MU_ERR_UNSUPPORTED_SIZE;
    cudaStream_t s = (cudaStream_t)stream;
    float* part_acc = scratch;
    float* part_ml = scratch + (long long)n_tokens * n_heads * maps * mu::MD_SPLITS * vdim;
    const int warps = group >= 4 ? 4 : group;                // a warp a head; more than four heads: in turns
    const dim3 grid(n_tokens, n_kv_heads, mu::MD_SPLITS), block(32 * warps);
    const dim3 mgrid(n_tokens, n_heads), mblock(vdim > 64 ? 128 : 64);
    typedef __nv_bfloat16 bf;
#define MU_MAPPED_DECODE(TE, M)                                                                                        \
    do {                                                                                                               \
        auto kernel = mu::mapped_decode_kernel<TE, M>;                                                                 \
        if (smem > 48 * 1024 &&                                                                                        \
            cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)       \
            return MU_ERR_LAUNCH;                                                                                      \
        const int code = mu::launch_pdl(kernel, grid, block, smem, s, 1, (const TE*)q, ldq, (const TE*)rows,           \
                                        block_table, max_pages, tok_pos, tok_seq, n_heads, n_kv_heads, dim, vdim,      \
                                        scale, window, vec, part_acc, part_ml, head_scale, chunk);                     \
        if (code != MU_OK) return code;                                                                                \
        return mu::launch_pdl(mu::mapped_merge_kernel<TE, M>, mgrid, mblock, (size_t)vdim * sizeof(float), s, 1,       \
                              (const float*)part_acc, (const float*)part_ml, n_heads, vdim, lambda, out_scale, eps,    \
                              unit_rms, (TE*)out, ldo, sink, (const TE*)gate, ldg);                                    \
    } while (0)
    if (is_bf16) {
        if (maps == 2) MU_MAPPED_DECODE(bf, 2);
        MU_MAPPED_DECODE(bf, 1);
    }
    if (maps == 2) MU_MAPPED_DECODE(float, 2);
    MU_MAPPED_DECODE(float, 1);
#undef MU_MAPPED_DECODE
}
