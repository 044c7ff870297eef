// Prompt steps of the attention with score maps (mapped_attention.cu says what it computes) on tensor cores,
// bfloat16: a block takes a tile of up to 64 consecutive tokens of one sequence and one head, and walks over the
// cache pages its tokens see.  A page's keys (both maps) and values of the head's kv head arrive by cp.async in two
// stages; per map S = Q K^T is mma.sync.m16n8k16 with float32 accumulators, the softmax runs in float32 on the
// accumulators (running maximum and sum per row), and P V follows with the SAME values for both maps.  The weights
// P enter that product as two bfloat16 terms (the rounded weight and what the rounding left), so they act with
// some 16 bits of mantissa instead of 8.  At the end a1 - lambda a2, the head's unit rms and the output scale, and
// the options of mapped_attention.cu (a multiplier per head on the scores, a sink in the denominator, a gate per head,
// chunks of positions instead of a window).
//
// Sizes: page of 64 positions; dim a multiple of 16 up to 256 per map; vdim a multiple of 16 up to 128; the cache
// row a multiple of 8 entries.  Anything else takes the CUDA-core kernel.
#include "common.cuh"

#include <math.h>

namespace mu {

constexpr int MM_TILE = 64;       // queries per block, keys per page
constexpr int MM_PAD = 8;         // entries between rows in shared memory: ldmatrix without bank conflicts

__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], const __nv_bfloat16* p) {
    const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void ldsm_x4_trans(uint32_t (&r)[4], const __nv_bfloat16* p) {
    const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void mma_bf16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ void cp_async16(void* dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src)
                 : "memory");
}

// VD: the head's value entries rounded up to 32, 64 or 128 (columns past vdim are zeros in shared memory).
template <int MAPS, int VD>
__global__ void __launch_bounds__(128, 1)
mapped_attention_mma_kernel(const __nv_bfloat16* __restrict__ q, long long ldq, const __nv_bfloat16* __restrict__ rows,
                            const int* __restrict__ block_table, int max_pages, const int* __restrict__ tok_pos,
                            const int* __restrict__ tok_seq, const int* __restrict__ tiles, int n_heads, int n_kv_heads,
                            int dim, int vdim, float scale, int window, float lambda, float out_scale, float eps,
                            int unit_rms, __nv_bfloat16* __restrict__ out, long long ldo,
                            const float* __restrict__ head_scale, int sink, const __nv_bfloat16* __restrict__ gate,
                            long long ldg, int chunk) {
    extern __shared__ __align__(16) unsigned char raw[];
    const int kw = MAPS * dim;                               // key entries of one kv head
    const int kp = kw + MM_PAD, vp = VD + MM_PAD;            // row pitches in shared memory
    __nv_bfloat16* qs = reinterpret_cast<__nv_bfloat16*>(raw);                 // [64][kp]
    __nv_bfloat16* ks = qs + MM_TILE * kp;                                     // [2][64][kp]
    __nv_bfloat16* vs = ks + 2 * MM_TILE * kp;                                 // [2][64][vp]
    pdl_trigger();
    pdl_wait();
    const int flat0 = tiles[2 * blockIdx.x], count = min(tiles[2 * blockIdx.x + 1], MM_TILE);
    const int h = blockIdx.y, g = h / (n_heads / n_kv_heads);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, gid = lane >> 2, tig = lane & 3;
    const int pos0 = tok_pos[flat0];
    if (head_scale) scale *= head_scale[h];
    const int* pages = block_table + (long long)tok_seq[flat0] * max_pages;
    const long long width = (long long)n_kv_heads * (kw + vdim);
    const long long key_off = (long long)g * kw, val_off = (long long)n_kv_heads * kw + (long long)g * vdim;
    const int last_key = pos0 + count - 1;
    // (with chunks: the first query's chunk starts first; a tile may reach into the next chunk)
    const int first_key = chunk > 0 ? pos0 - pos0 % chunk : window > 0 ? max(0, pos0 - window + 1) : 0;
    const int page_lo = first_key / MM_TILE, page_hi = last_key / MM_TILE;

    // the value columns past vdim stay zero; the queries of the tile (rows past count are zeros)
    for (int i = tid; i < 2 * MM_TILE * vp; i += blockDim.x) vs[i] = __float2bfloat16_rn(0.0f);
    const int qchunks = kw / 8;
    for (int i = tid; i < MM_TILE * qchunks; i += blockDim.x) {
        const int r = i / qchunks, c = (i % qchunks) * 8;
        uint4 v = make_uint4(0u, 0u, 0u, 0u);
        if (r < count) v = *reinterpret_cast<const uint4*>(q + (long long)(flat0 + r) * ldq + (long long)h * kw + c);
        *reinterpret_cast<uint4*>(qs + r * kp + c) = v;
    }
    __syncthreads();                                         // the zeros are in place before any copy lands on them

    const int vchunks = vdim / 8;
    auto load_page = [&](int page_index, int stage) {
        const __nv_bfloat16* src = rows + (long long)pages[page_index] * MM_TILE * width;
        __nv_bfloat16* kd = ks + stage * MM_TILE * kp;
        __nv_bfloat16* vd = vs + stage * MM_TILE * vp;
        for (int i = tid; i < MM_TILE * (qchunks + vchunks); i += blockDim.x) {
            const int r = i / (qchunks + vchunks), c = i % (qchunks + vchunks);
            if (c < qchunks) cp_async16(kd + r * kp + c * 8, src + r * width + key_off + c * 8);
            else cp_async16(vd + r * vp + (c - qchunks) * 8, src + r * width + val_off + (c - qchunks) * 8);
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };

    float o[MAPS][VD / 8][4];
    float m_run[MAPS][2], l_run[MAPS][2];
#pragma unroll
    for (int a = 0; a < MAPS; ++a) {
        m_run[a][0] = m_run[a][1] = -INFINITY;
        l_run[a][0] = l_run[a][1] = 0.0f;
#pragma unroll
        for (int j = 0; j < VD / 8; ++j) o[a][j][0] = o[a][j][1] = o[a][j][2] = o[a][j][3] = 0.0f;
    }
    const int row0 = warp * 16 + gid;                        // this thread's two rows of the tile: row0 and row0 + 8
    const int qpos[2] = {pos0 + row0, pos0 + row0 + 8};
    const bool real[2] = {row0 < count, row0 + 8 < count};

    load_page(page_lo, 0);
    for (int pg = page_lo; pg <= page_hi; ++pg) {
        const int stage = (pg - page_lo) & 1;
        if (pg < page_hi) {
            load_page(pg + 1, stage ^ 1);
            asm volatile("cp.async.wait_group 1;" ::: "memory");
        } else {
            asm volatile("cp.async.wait_group 0;" ::: "memory");
        }
        __syncthreads();
        const __nv_bfloat16* kt = ks + stage * MM_TILE * kp;
        const __nv_bfloat16* vt = vs + stage * MM_TILE * vp;
        const int key0 = pg * MM_TILE;
        // a warp whose 16 queries see nothing of this page skips it (a page wholly after them, or wholly before their windows)
        const int w_first = pos0 + warp * 16, w_last = min(pos0 + warp * 16 + 15, last_key);
        const bool skip = key0 > w_last || warp * 16 >= count ||
                          (chunk > 0 ? key0 + MM_TILE - 1 < w_first - w_first % chunk
                                     : window > 0 && key0 + MM_TILE - 1 < w_first - window + 1);
        if (!skip) {
#pragma unroll
            for (int a = 0; a < MAPS; ++a) {
                float s[8][4];
#pragma unroll
                for (int j = 0; j < 8; ++j) s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.0f;
                for (int kk = 0; kk < dim / 16; ++kk) {
                    uint32_t af[4];
                    ldsm_x4(af, qs + (warp * 16 + (lane & 15)) * kp + a * dim + kk * 16 + (lane >> 4) * 8);
#pragma unroll
                    for (int j = 0; j < 8; j += 2) {
                        uint32_t bf[4];
                        ldsm_x4(bf, kt + (j * 8 + (lane & 7) + (lane >> 4) * 8) * kp + a * dim + kk * 16 + ((lane >> 3) & 1) * 8);
                        mma_bf16(s[j], af, bf[0], bf[1]);
                        mma_bf16(s[j + 1], af, bf[2], bf[3]);
                    }
                }
                // scale, mask, running maximum
                float top[2] = {-INFINITY, -INFINITY};
#pragma unroll
                for (int j = 0; j < 8; ++j)
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const int r = e >> 1, kj = key0 + j * 8 + tig * 2 + (e & 1);
                        const bool seen = real[r] && kj <= qpos[r] &&
                                          (chunk > 0 ? kj >= qpos[r] - qpos[r] % chunk : window == 0 || qpos[r] - kj < window);
                        s[j][e] = seen ? s[j][e] * scale : -INFINITY;
                        top[r] = fmaxf(top[r], s[j][e]);
                    }
                float corr[2];
#pragma unroll
                for (int r = 0; r < 2; ++r) {
                    top[r] = fmaxf(top[r], __shfl_xor_sync(0xffffffffu, top[r], 1));
                    top[r] = fmaxf(top[r], __shfl_xor_sync(0xffffffffu, top[r], 2));
                    const float m_new = fmaxf(m_run[a][r], top[r]);
                    corr[r] = m_new == -INFINITY ? 1.0f : expf(m_run[a][r] - m_new);
                    m_run[a][r] = m_new;
                    l_run[a][r] *= corr[r];
                }
#pragma unroll
                for (int j = 0; j < VD / 8; ++j) {
                    o[a][j][0] *= corr[0]; o[a][j][1] *= corr[0];
                    o[a][j][2] *= corr[1]; o[a][j][3] *= corr[1];
                }
                uint32_t ph[4][4], pl[4][4];                 // P as A fragments of the four 16-key steps: rounded, and the rest
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    float p[4];
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const int r = e >> 1;
                        p[e] = s[j][e] == -INFINITY ? 0.0f : expf(s[j][e] - m_run[a][r]);
                        l_run[a][r] += p[e];
                    }
                    const uint32_t h01 = pack_bf16(p[0], p[1]), h23 = pack_bf16(p[2], p[3]);
                    const __nv_bfloat162 b01 = *reinterpret_cast<const __nv_bfloat162*>(&h01);
                    const __nv_bfloat162 b23 = *reinterpret_cast<const __nv_bfloat162*>(&h23);
                    const uint32_t l01 = pack_bf16(p[0] - __low2float(b01), p[1] - __high2float(b01));
                    const uint32_t l23 = pack_bf16(p[2] - __low2float(b23), p[3] - __high2float(b23));
                    ph[j >> 1][(j & 1) * 2] = h01; ph[j >> 1][(j & 1) * 2 + 1] = h23;
                    pl[j >> 1][(j & 1) * 2] = l01; pl[j >> 1][(j & 1) * 2 + 1] = l23;
                }
#pragma unroll
                for (int kk = 0; kk < 4; ++kk) {
#pragma unroll
                    for (int j = 0; j < VD / 8; j += 2) {
                        uint32_t bf[4];
                        ldsm_x4_trans(bf, vt + (kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * vp + j * 8 + (lane >> 4) * 8);
                        mma_bf16(o[a][j], ph[kk], bf[0], bf[1]);
                        mma_bf16(o[a][j], pl[kk], bf[0], bf[1]);
                        mma_bf16(o[a][j + 1], ph[kk], bf[2], bf[3]);
                        mma_bf16(o[a][j + 1], pl[kk], bf[2], bf[3]);
                    }
                }
            }
        }
        __syncthreads();                                     // everyone is done with this stage before it is refilled
    }

    // sums of the rows over the four threads that share them, then the maps' difference, the unit rms, the store
    float inv_l[MAPS][2];
#pragma unroll
    for (int a = 0; a < MAPS; ++a)
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            float l = l_run[a][r];
            l += __shfl_xor_sync(0xffffffffu, l, 1);
            l += __shfl_xor_sync(0xffffffffu, l, 2);
            if (sink) {
                // one more key of score zero and no value: sums and maximum move to max(m, 0)
                const float top = fmaxf(m_run[a][r], 0.0f);
                const float f = m_run[a][r] == -INFINITY ? 0.0f : expf(m_run[a][r] - top);
                inv_l[a][r] = f / (l * f + expf(-top));
            } else {
                inv_l[a][r] = l > 0.0f ? 1.0f / l : 0.0f;
            }
        }
    float sq[2] = {0.0f, 0.0f};
#pragma unroll
    for (int j = 0; j < VD / 8; ++j)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int r = e >> 1;
            float v = o[0][j][e] * inv_l[0][r];
            if (MAPS == 2) v -= lambda * (o[MAPS - 1][j][e] * inv_l[MAPS - 1][r]);
            o[0][j][e] = v;
            sq[r] += v * v;                                  // (columns past vdim are zeros)
        }
    float mult[2] = {out_scale, out_scale};
    if (unit_rms) {
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            sq[r] += __shfl_xor_sync(0xffffffffu, sq[r], 1);
            sq[r] += __shfl_xor_sync(0xffffffffu, sq[r], 2);
            mult[r] *= 1.0f / sqrtf(sq[r] / (float)vdim + eps);
        }
    }
    if (gate) {
#pragma unroll
        for (int r = 0; r < 2; ++r)
            if (real[r]) mult[r] *= 1.0f / (1.0f + expf(-__bfloat162float(gate[(long long)(flat0 + row0 + 8 * r) * ldg + h])));
    }
#pragma unroll
    for (int j = 0; j < VD / 8; ++j) {
        const int col = j * 8 + tig * 2;
        if (col < vdim) {
#pragma unroll
            for (int r = 0; r < 2; ++r)
                if (real[r]) {
                    __nv_bfloat16* dst = out + (long long)(flat0 + row0 + 8 * r) * ldo + (long long)h * vdim + col;
                    *reinterpret_cast<__nv_bfloat162*>(dst) =
                        __floats2bfloat162_rn(o[0][j][2 * r] * mult[r], o[0][j][2 * r + 1] * mult[r]);
                }
        }
    }
}

}  // namespace mu

// Whether the tensor-core kernel takes these sizes (page of 64 positions assumed by the caller's check).
MU_EXPORT int mu_mapped_attention_mma_fits(int n_kv_heads, int maps, int dim, int vdim, int page_tokens) {
    const long long width = (long long)n_kv_heads * (maps * dim + vdim);
    return page_tokens == mu::MM_TILE && (maps == 1 || maps == 2) && dim % 16 == 0 && dim > 0 && dim <= 256 &&
           vdim % 16 == 0 && vdim > 0 && vdim <= 128 && width % 8 == 0;
}

MU_EXPORT int mu_mapped_attention_mma(const void* q, long long ldq, const void* rows, const int* block_table,
                                      int max_pages, int page_tokens, const int* tok_pos, const int* tok_seq,
                                      const int* tiles, int n_tiles, int n_heads, int n_kv_heads, int maps, int dim,
                                      int vdim, float scale, int window, float lambda, float out_scale, float eps,
                                      int unit_rms, void* out, long long ldo, void* stream, const float* head_scale,
                                      int sink, const void* gate, long long ldg, int chunk) {
    if (n_tiles <= 0) return MU_OK;
    if (!q || !rows || !block_table || !tok_pos || !tok_seq || !tiles || !out || n_heads <= 0 || n_kv_heads <= 0 ||
        n_heads % n_kv_heads || window < 0 || chunk < 0)
        return MU_ERR_BAD_ARGUMENT;
    if (!mu_mapped_attention_mma_fits(n_kv_heads, maps, dim, vdim, page_tokens)) return MU_ERR_UNSUPPORTED_SIZE;
    if (((uintptr_t)q & 15) || ((uintptr_t)rows & 15) || ((uintptr_t)out & 3) || ldq % 8 || ldo % 2)
        return MU_ERR_ALIGNMENT;
    const int vd = vdim <= 32 ? 32 : vdim <= 64 ? 64 : 128;
    const size_t smem = ((size_t)3 * mu::MM_TILE * (maps * dim + mu::MM_PAD) + (size_t)2 * mu::MM_TILE * (vd + mu::MM_PAD)) *
                        sizeof(__nv_bfloat16);
    if (smem > 220 * 1024) return MU_ERR_UNSUPPORTED_SIZE;
    cudaStream_t s = (cudaStream_t)stream;
    const dim3 grid(n_tiles, n_heads), block(128);
    typedef __nv_bfloat16 bf;
#define MU_MAPPED_MMA(M, VD)                                                                                           \
    do {                                                                                                               \
        auto kernel = mu::mapped_attention_mma_kernel<M, VD>;                                                          \
        if (smem > 48 * 1024 &&                                                                                        \
            cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)       \
            return MU_ERR_LAUNCH;                                                                                      \
        return mu::launch_pdl(kernel, grid, block, smem, s, 1, (const bf*)q, ldq, (const bf*)rows, block_table,        \
                              max_pages, tok_pos, tok_seq, tiles, n_heads, n_kv_heads, dim, vdim, scale, window,       \
                              lambda, out_scale, eps, unit_rms, (bf*)out, ldo, head_scale, sink, (const bf*)gate, ldg, \
                              chunk);                                                                                  \
    } while (0)
    if (maps == 2) {
        if (vd == 32) MU_MAPPED_MMA(2, 32);
        if (vd == 64) MU_MAPPED_MMA(2, 64);
        MU_MAPPED_MMA(2, 128);
    }
    if (vd == 32) MU_MAPPED_MMA(1, 32);
    if (vd == 64) MU_MAPPED_MMA(1, 64);
    MU_MAPPED_MMA(1, 128);
#undef MU_MAPPED_MMA
}
