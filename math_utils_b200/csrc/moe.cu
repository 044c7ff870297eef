// A feed-forward of routed experts: router, grouping of (token, expert) pairs by expert, the experts'
// products over each expert's rows, and the weighted sum per token.  Nothing is read back by the host,
// so a step with these kernels can be recorded in a CUDA graph: grids are sized for the worst case and
// blocks without work leave at once.
//
// mu_moe_route    z = W_r h in float32; s = sigmoid(z) (or softmax over the experts); the `top` experts with
//                 the largest s + correction are chosen (ties: the lower index); weight = s * scale
//                 (optionally divided by the chosen experts' sum).  A block per token, or per eight in prompt steps.
// mu_moe_group    counts the pairs of each expert, gives every pair a slot so that an expert's slots are
//                 contiguous, and lists tiles of TM slots that never straddle two experts.
// mu_moe_gemm     for every tile: out[slot, :] = act(W1[e] x[row]) (* W2[e] x[row]) on CUDA cores, one running
//                 sum per output over k in order, so a row's result does not depend on which rows share its
//                 tile.  Rows of x are gathered through the slot's pair (token = pair / top) or are the slots
//                 themselves.
// mu_moe_combine  y[t, :] = sum over the token's pairs, in the order of its choices, of weight * out[slot, :].
//
// Options for other designs.  Identity experts: the router's outputs from `n_real` on have no matrices; their
// pairs get no slot (slot_of = -1) and no tile, and the combine takes the token's own input row for them.  The
// router can divide the chosen weights by (their sum + renorm_eps), and compute one more number per token,
// sigmoid(gate_w . h), which the combine multiplies a shared expert's row by before adding it.  The experts'
// product takes an activation code (mu::ACT_*) for experts of the form W2 act(W1 x).  The combine can add its
// result to what `out` holds.
#include "common.cuh"

#include <math.h>

namespace mu {

constexpr int MOE_TM = 32, MOE_TN = 64, MOE_TK = 32;

constexpr int ROUTE_WARPS = 16;

// A block takes TOK consecutive tokens: their rows are staged in shared memory as float32, the warps share the
// experts (each logit one warp's sum over the row, lanes striding along it; a router row is read once for the
// block's tokens), then warp i scores and chooses for token i.  A token's sums run in the same order whatever TOK
// is and whichever tokens share its block.
template <typename T, int TOK>
__global__ void __launch_bounds__(ROUTE_WARPS * 32)
moe_route_kernel(const T* __restrict__ h, long long ldh, const float* __restrict__ router,
                 const float* __restrict__ correction, int n_tokens, int hidden, int n_experts, int top,
                 float scale, int softmax, int renormalize, int* __restrict__ expert_of,
                 float* __restrict__ weight_of, float renorm_eps, const float* __restrict__ gate_w,
                 float* __restrict__ gate_out) {
    extern __shared__ __align__(16) float sm[];        // rows [TOK][hidden], scores [TOK][n_experts], choice [TOK][n_experts]
    pdl_trigger();
    pdl_wait();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int t0 = blockIdx.x * TOK, nt = min(TOK, n_tokens - t0);
    float* hrow = sm;
    float* score_all = sm + (size_t)TOK * hidden;
    float* choice_all = score_all + TOK * n_experts;
    if (sizeof(T) == 2 && hidden % 8 == 0 && ldh % 8 == 0 && ((uintptr_t)h & 15) == 0) {
        // eight bfloat16 entries a thread and load
        const int pieces = hidden / 8;
        for (int j = threadIdx.x; j < TOK * pieces; j += blockDim.x) {
            const int i = j / pieces, c = j % pieces;
            uint4 raw = make_uint4(0u, 0u, 0u, 0u);
            if (i < nt) raw = *reinterpret_cast<const uint4*>(h + (long long)(t0 + i) * ldh + 8 * c);
            const __nv_bfloat162* p2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
            float4* dst = reinterpret_cast<float4*>(hrow + i * hidden + 8 * c);
            const float2 a = __bfloat1622float2(p2[0]), b = __bfloat1622float2(p2[1]);
            const float2 c2 = __bfloat1622float2(p2[2]), d2 = __bfloat1622float2(p2[3]);
            dst[0] = make_float4(a.x, a.y, b.x, b.y);
            dst[1] = make_float4(c2.x, c2.y, d2.x, d2.y);
        }
    } else {
        for (int i = 0; i < TOK; ++i) {
            const T* row = h + (long long)(t0 + i) * ldh;
            for (int d = threadIdx.x; d < hidden; d += blockDim.x) hrow[i * hidden + d] = i < nt ? to_float(row[d]) : 0.0f;
        }
    }
    __syncthreads();
    const bool wide = hidden % 4 == 0 && ((uintptr_t)router & 15) == 0 &&
                      ((uintptr_t)gate_w & 15) == 0;                          // rows of the router in 16-byte pieces
    // (with gate_w: one more sum, over the shared expert's gate row, by the warp whose turn it is)
    for (int e = warp; e < n_experts + (gate_w ? 1 : 0); e += ROUTE_WARPS) {
        const float* w = e < n_experts ? router + (long long)e * hidden : gate_w;
        float z[TOK];
        if (wide) {
            const float4* w4 = reinterpret_cast<const float4*>(w);
            const float4* h4 = reinterpret_cast<const float4*>(hrow);
            const int n4 = hidden / 4;
            float z0[TOK], z1[TOK], z2[TOK], z3[TOK];                        // a lane's sum in four parts, then in order
#pragma unroll
            for (int i = 0; i < TOK; ++i) z0[i] = z1[i] = z2[i] = z3[i] = 0.0f;
#pragma unroll 8
            for (int d = lane; d < n4; d += 32) {                            // (unrolled: the row's loads go out together)
                const float4 b = w4[d];
#pragma unroll
                for (int i = 0; i < TOK; ++i) {
                    const float4 a = h4[i * n4 + d];
                    z0[i] += a.x * b.x; z1[i] += a.y * b.y; z2[i] += a.z * b.z; z3[i] += a.w * b.w;
                }
            }
#pragma unroll
            for (int i = 0; i < TOK; ++i) z[i] = (z0[i] + z1[i]) + (z2[i] + z3[i]);
        } else {
#pragma unroll
            for (int i = 0; i < TOK; ++i) z[i] = 0.0f;
            for (int d = lane; d < hidden; d += 32) {
                const float b = w[d];
#pragma unroll
                for (int i = 0; i < TOK; ++i) z[i] += hrow[i * hidden + d] * b;
            }
        }
#pragma unroll
        for (int i = 0; i < TOK; ++i) {
            const float zi = warp_sum(z[i]);
            if (lane == 0 && i < nt) {
                if (e < n_experts) score_all[i * n_experts + e] = zi;
                else gate_out[t0 + i] = 1.0f / (1.0f + expf(-zi));
            }
        }
    }
    __syncthreads();
    if (warp >= nt) return;
    const int t = t0 + warp;
    float* score = score_all + warp * n_experts;
    float* choice = choice_all + warp * n_experts;
    if (softmax) {
        float top_z = -INFINITY, sum = 0.0f;
        for (int e = lane; e < n_experts; e += 32) top_z = fmaxf(top_z, score[e]);
        top_z = warp_max(top_z);
        for (int e = lane; e < n_experts; e += 32) sum += expf(score[e] - top_z);
        sum = warp_sum(sum);
        for (int e = lane; e < n_experts; e += 32) score[e] = expf(score[e] - top_z) / sum;
    } else {
        for (int e = lane; e < n_experts; e += 32) score[e] = 1.0f / (1.0f + expf(-score[e]));
    }
    for (int e = lane; e < n_experts; e += 32) choice[e] = score[e] + (correction ? correction[e] : 0.0f);
    __syncwarp();
    float kept = 0.0f;
    for (int k = 0; k < top; ++k) {
        float best = -INFINITY;
        int arg = n_experts;
        for (int e = lane; e < n_experts; e += 32)
            if (choice[e] > best) { best = choice[e]; arg = e; }       // first maximum of the lane's experts
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oa = __shfl_xor_sync(0xffffffffu, arg, o);
            if (ob > best || (ob == best && oa < arg)) { best = ob; arg = oa; }
        }
        if (arg >= n_experts) arg = 0;                                 // (not a number everywhere)
        if (lane == 0) {
            expert_of[(long long)t * top + k] = arg;
            weight_of[(long long)t * top + k] = score[arg];
            choice[arg] = -INFINITY;
        }
        kept += score[arg];
        __syncwarp();
    }
    const float f = renormalize ? scale / (kept + renorm_eps) : scale;
    for (int k = lane; k < top; k += 32) weight_of[(long long)t * top + k] *= f;
}

// One block.  slot_of[pair], pair_of[slot], and the tile list: tile_info[3 i] = expert, [3 i + 1] = first slot,
// [3 i + 2] = rows; n_tiles[0] = how many.
__global__ void moe_group_kernel(const int* __restrict__ expert_of, int n_pairs, int n_experts, int* __restrict__ slot_of,
                                 int* __restrict__ pair_of, int* __restrict__ tile_info, int* __restrict__ n_tiles,
                                 int tile_rows, int n_real) {
    extern __shared__ int smi[];                       // count [n_experts], first [n_experts + 1], tile0 [n_experts + 1]
    int* count = smi;
    int* first = smi + n_experts;
    int* tile0 = first + n_experts + 1;
    pdl_trigger();
    pdl_wait();
    for (int e = threadIdx.x; e < n_experts; e += blockDim.x) count[e] = 0;
    __syncthreads();
    for (int p = threadIdx.x; p < n_pairs; p += blockDim.x)
        if (expert_of[p] < n_real) atomicAdd(&count[expert_of[p]], 1);
    __syncthreads();
    if (threadIdx.x == 0) {
        int at = 0, tiles = 0;
        for (int e = 0; e < n_experts; ++e) {
            first[e] = at;
            tile0[e] = tiles;
            at += count[e];
            tiles += (count[e] + tile_rows - 1) / tile_rows;
        }
        first[n_experts] = at;
        tile0[n_experts] = tiles;
        n_tiles[0] = tiles;
    }
    __syncthreads();
    for (int e = threadIdx.x; e < n_experts; e += blockDim.x) {
        const int n = count[e];
        for (int i = 0, k = tile0[e]; i < n; i += tile_rows, ++k) {
            tile_info[3 * k] = e;
            tile_info[3 * k + 1] = first[e] + i;
            tile_info[3 * k + 2] = min(tile_rows, n - i);
        }
        count[e] = 0;                                  // now the cursor within the expert's slots
    }
    __syncthreads();
    // slots in the order of the pairs within each expert: a thread takes a run of pairs, runs in thread order
    // would need a scan per expert; the order within an expert changes no result (every row is computed by
    // itself), so the slots are simply drawn
    for (int p = threadIdx.x; p < n_pairs; p += blockDim.x) {
        const int e = expert_of[p];
        if (e >= n_real) {                             // an identity expert: nothing to compute
            slot_of[p] = -1;
            continue;
        }
        const int slot = first[e] + atomicAdd(&count[e], 1);
        slot_of[p] = slot;
        pair_of[slot] = p;
    }
}

__device__ __forceinline__ float silu(float z) { return z / (1.0f + expf(-z)); }

// GATED: out = silu(W1 x) * (W2 x); else out = W1 x.  x rows: pair_of[slot] / top if pair_of, else slot.
template <typename T, typename TO, bool GATED>
__global__ void __launch_bounds__(256)
moe_gemm_kernel(const T* __restrict__ x, long long ldx, const int* __restrict__ pair_of, int top,
                const T* __restrict__ w1, const T* __restrict__ w2, long long expert_stride, long long ldw,
                const int* __restrict__ tile_info, const int* __restrict__ n_tiles, int n, int k,
                TO* __restrict__ out, long long ldo, int act) {
    __shared__ float sa[MOE_TM][MOE_TK + 1];
    __shared__ float sw1[MOE_TN][MOE_TK + 1];
    __shared__ float sw2[GATED ? MOE_TN : 1][MOE_TK + 1];
    __shared__ int src_row[MOE_TM];
    pdl_trigger();
    pdl_wait();
    const int tile = blockIdx.x;
    if (tile >= n_tiles[0]) return;
    const int e = tile_info[3 * tile], slot0 = tile_info[3 * tile + 1], rows = tile_info[3 * tile + 2];
    const int n0 = blockIdx.y * MOE_TN;
    const T* w1e = w1 + (long long)e * expert_stride;
    const T* w2e = GATED ? w2 + (long long)e * expert_stride : nullptr;
    if (threadIdx.x < MOE_TM) {
        const int r = threadIdx.x;
        src_row[r] = r < rows ? (pair_of ? pair_of[slot0 + r] / top : slot0 + r) : -1;
    }
    __syncthreads();
    const int ty = threadIdx.x / 16, tx = threadIdx.x % 16;     // rows 2 ty, 2 ty + 1; columns tx + 16 j
    float a1[2][4] = {}, a2[2][4] = {};
    for (int k0 = 0; k0 < k; k0 += MOE_TK) {
        for (int i = threadIdx.x; i < MOE_TM * MOE_TK; i += 256) {
            const int r = i / MOE_TK, c = i % MOE_TK;
            const int row = src_row[r];
            sa[r][c] = (row >= 0 && k0 + c < k) ? to_float(x[(long long)row * ldx + k0 + c]) : 0.0f;
        }
        for (int i = threadIdx.x; i < MOE_TN * MOE_TK; i += 256) {
            const int r = i / MOE_TK, c = i % MOE_TK;
            const bool in = n0 + r < n && k0 + c < k;
            sw1[r][c] = in ? to_float(w1e[(long long)(n0 + r) * ldw + k0 + c]) : 0.0f;
            if (GATED) sw2[r][c] = in ? to_float(w2e[(long long)(n0 + r) * ldw + k0 + c]) : 0.0f;
        }
        __syncthreads();
#pragma unroll 8
        for (int c = 0; c < MOE_TK; ++c) {
            const float x0 = sa[2 * ty][c], x1 = sa[2 * ty + 1][c];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float u = sw1[tx + 16 * j][c];
                a1[0][j] += x0 * u;
                a1[1][j] += x1 * u;
                if (GATED) {
                    const float v = sw2[tx + 16 * j][c];
                    a2[0][j] += x0 * v;
                    a2[1][j] += x1 * v;
                }
            }
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int r = 2 * ty + i;
        if (r >= rows) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int col = n0 + tx + 16 * j;
            if (col >= n) continue;
            const float v = GATED ? silu(a1[i][j]) * a2[i][j] : apply_act(a1[i][j], act);
            out[(long long)(slot0 + r) * ldo + col] = from_float<TO>(v);
        }
    }
}

// x (may be null): the rows the experts read, for pairs without a slot; shared / shared_gate (may be null): a row
// per token that every token gets, times the token's gate.
template <typename TX>
__global__ void moe_combine_kernel(const float* __restrict__ y, long long ldy, const int* __restrict__ slot_of,
                                   const float* __restrict__ weight_of, int top, int width, float* __restrict__ out,
                                   long long ldo, const TX* __restrict__ x, long long ldx,
                                   const float* __restrict__ shared, long long lds,
                                   const float* __restrict__ shared_gate, int add) {
    pdl_trigger();
    pdl_wait();
    const int t = blockIdx.x;
    for (int d = threadIdx.x; d < width; d += blockDim.x) {
        float v = 0.0f;
        for (int k = 0; k < top; ++k) {
            const int slot = slot_of[(long long)t * top + k];
            const float row = slot >= 0 ? y[(long long)slot * ldy + d] : to_float(x[(long long)t * ldx + d]);
            v += weight_of[(long long)t * top + k] * row;
        }
        if (shared) v += (shared_gate ? shared_gate[t] : 1.0f) * shared[(long long)t * lds + d];
        if (add) v += out[(long long)t * ldo + d];
        out[(long long)t * ldo + d] = v;
    }
}

__device__ __forceinline__ float4 load4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float4 load4(const __nv_bfloat16* p) {
    const uint2 raw = *reinterpret_cast<const uint2*>(p);
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
    const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
    return make_float4(a.x, a.y, b.x, b.y);
}

// The same for rows that are whole 16-byte pieces: four entries a thread, every row's piece asked for before the
// first is used.  TOP > 0: the number of choices at compile time (the loads of all choices are in flight together).
template <typename TX, int TOP>
__global__ void moe_combine_vec_kernel(const float* __restrict__ y, long long ldy, const int* __restrict__ slot_of,
                                       const float* __restrict__ weight_of, int top, int width, float* __restrict__ out,
                                       long long ldo, const TX* __restrict__ x, long long ldx,
                                       const float* __restrict__ shared, long long lds,
                                       const float* __restrict__ shared_gate, int add) {
    pdl_trigger();
    pdl_wait();
    const int t = blockIdx.x;
    if (TOP > 0) top = TOP;
    for (int d = 4 * threadIdx.x; d < width; d += 4 * blockDim.x) {
        float4 v = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        if (TOP > 0) {
            float4 row[TOP > 0 ? TOP : 1];
            float w[TOP > 0 ? TOP : 1];
#pragma unroll
            for (int k = 0; k < TOP; ++k) {
                const int slot = slot_of[(long long)t * TOP + k];
                w[k] = weight_of[(long long)t * TOP + k];
                row[k] = slot >= 0 ? load4(y + (long long)slot * ldy + d) : load4(x + (long long)t * ldx + d);
            }
#pragma unroll
            for (int k = 0; k < TOP; ++k) {                                // in the order of the choices
                v.x += w[k] * row[k].x; v.y += w[k] * row[k].y; v.z += w[k] * row[k].z; v.w += w[k] * row[k].w;
            }
        } else {
            for (int k = 0; k < top; ++k) {
                const int slot = slot_of[(long long)t * top + k];
                const float w = weight_of[(long long)t * top + k];
                const float4 row = slot >= 0 ? load4(y + (long long)slot * ldy + d) : load4(x + (long long)t * ldx + d);
                v.x += w * row.x; v.y += w * row.y; v.z += w * row.z; v.w += w * row.w;
            }
        }
        if (shared) {
            const float g = shared_gate ? shared_gate[t] : 1.0f;
            const float4 sh = load4(shared + (long long)t * lds + d);
            v.x += g * sh.x; v.y += g * sh.y; v.z += g * sh.z; v.w += g * sh.w;
        }
        float* dst = out + (long long)t * ldo + d;
        if (add) {
            const float4 old = load4(dst);
            v.x += old.x; v.y += old.y; v.z += old.z; v.w += old.w;
        }
        *reinterpret_cast<float4*>(dst) = v;
    }
}

// The same sum, normed and added into the residual stream: out[t, :] += tanh(alpha v) w + b with v the token's sum.
__global__ void moe_combine_tanh_kernel(const float* __restrict__ y, long long ldy, const int* __restrict__ slot_of,
                                        const float* __restrict__ weight_of, int top, int width,
                                        const float* __restrict__ w, const float* __restrict__ b,
                                        const float* __restrict__ alpha, float* __restrict__ out, long long ldo) {
    pdl_trigger();
    pdl_wait();
    const int t = blockIdx.x;
    const float a = alpha[0];
    for (int d = threadIdx.x; d < width; d += blockDim.x) {
        float v = 0.0f;
        for (int k = 0; k < top; ++k)
            v += weight_of[(long long)t * top + k] * y[(long long)slot_of[(long long)t * top + k] * ldy + d];
        out[(long long)t * ldo + d] += tanhf(a * v) * w[d] + (b ? b[d] : 0.0f);
    }
}

}  // namespace mu

MU_EXPORT int mu_moe_combine_tanh(const float* y, long long ldy, const int* slot_of, const float* weight_of, int n_tokens,
                                  int top, int width, const float* w, const float* b, const float* alpha, float* out,
                                  long long ldo, void* stream) {
    if (n_tokens <= 0) return MU_OK;
    if (!y || !slot_of || !weight_of || !out || !w || !alpha || top <= 0 || width <= 0) return MU_ERR_BAD_ARGUMENT;
    return mu::launch_pdl(mu::moe_combine_tanh_kernel, dim3(n_tokens), dim3(width >= 1024 ? 256 : 128), 0,
                          (cudaStream_t)stream, 1, y, ldy, slot_of, weight_of, top, width, w, b, alpha, out, ldo);
}

MU_EXPORT int mu_moe_tile_rows() { return mu::MOE_TM; }

MU_EXPORT int mu_moe_route(const void* h, long long ldh, int h_bf16, const float* router, const float* correction,
                           int n_tokens, int hidden, int n_experts, int top, float scale, int softmax, int renormalize,
                           int* expert_of, float* weight_of, void* stream, float renorm_eps, const float* gate_w,
                           float* gate_out) {
    if (n_tokens <= 0) return MU_OK;
    if (!h || !router || !expert_of || !weight_of || hidden <= 0 || n_experts <= 0 || top <= 0 || top > n_experts ||
        (gate_w != nullptr) != (gate_out != nullptr))
        return MU_ERR_BAD_ARGUMENT;
    // prompt steps: several tokens a block, so that the router's rows are read once for all of them (with a block a
    // token the router came out of the L2 once per token); few tokens: a block each, spread over the SMs
    int tok = n_tokens >= 4 * mu::sm_count() ? 8 : 1;
    while (tok > 1 && (size_t)tok * (hidden + 2 * n_experts) * sizeof(float) > 48 * 1024) tok /= 2;
    const size_t smem = (size_t)tok * (hidden + 2 * n_experts) * sizeof(float);
    if (smem > 48 * 1024) return MU_ERR_UNSUPPORTED_SIZE;
    cudaStream_t s = (cudaStream_t)stream;
    const dim3 grid((n_tokens + tok - 1) / tok), block(mu::ROUTE_WARPS * 32);
#define MU_ROUTE(T, TOK)                                                                                               \
    return mu::launch_pdl(mu::moe_route_kernel<T, TOK>, grid, block, smem, s, 1, (const T*)h, ldh, router, correction, \
                          n_tokens, hidden, n_experts, top, scale, softmax, renormalize, expert_of, weight_of,         \
                          renorm_eps, gate_w, gate_out)
    if (h_bf16) {
        if (tok == 8) MU_ROUTE(__nv_bfloat16, 8);
        if (tok == 4) MU_ROUTE(__nv_bfloat16, 4);
        if (tok == 2) MU_ROUTE(__nv_bfloat16, 2);
        MU_ROUTE(__nv_bfloat16, 1);
    }
    if (tok == 8) MU_ROUTE(float, 8);
    if (tok == 4) MU_ROUTE(float, 4);
    if (tok == 2) MU_ROUTE(float, 2);
    MU_ROUTE(float, 1);
#undef MU_ROUTE
}

// tile_info needs 3 * (n_pairs / tile_rows + n_experts) ints.  tile_rows: the CUDA-core product takes tiles of
// mu_moe_tile_rows() slots, the tensor-core product of 32 or 64.
// n_real (0: all of them): experts from n_real on are identity experts.
MU_EXPORT int mu_moe_group(const int* expert_of, int n_pairs, int n_experts, int* slot_of, int* pair_of, int* tile_info,
                           int* n_tiles, int tile_rows, void* stream, int n_real) {
    if (n_pairs <= 0) return MU_OK;
    if (!expert_of || !slot_of || !pair_of || !tile_info || !n_tiles || n_experts <= 0 || tile_rows <= 0)
        return MU_ERR_BAD_ARGUMENT;
    const size_t smem = (size_t)(3 * n_experts + 2) * sizeof(int);
    if (smem > 48 * 1024) return MU_ERR_UNSUPPORTED_SIZE;
    if (n_real < 0 || n_real > n_experts) return MU_ERR_BAD_ARGUMENT;
    return mu::launch_pdl(mu::moe_group_kernel, dim3(1), dim3(1024), smem, (cudaStream_t)stream, 1, expert_of, n_pairs,
                          n_experts, slot_of, pair_of, tile_info, n_tiles, tile_rows, n_real > 0 ? n_real : n_experts);
}

// w1 (and w2 when gated): [n_experts][n][k] with row stride ldw and expert stride `expert_stride` elements.
// max_tiles: the bound the grid is sized for (n_pairs / tile_rows + n_experts covers every grouping).
MU_EXPORT int mu_moe_gemm(const void* x, long long ldx, const int* pair_of, int top, const void* w1, const void* w2,
                          long long expert_stride, long long ldw, const int* tile_info, const int* n_tiles,
                          int max_tiles, int n, int k, void* out, long long ldo, int is_bf16, int out_bf16,
                          void* stream, int act) {
    if (max_tiles <= 0) return MU_OK;
    if (!x || !w1 || !tile_info || !n_tiles || !out || n <= 0 || k <= 0 || (pair_of && top <= 0))
        return MU_ERR_BAD_ARGUMENT;
    if (is_bf16 != out_bf16 && !(is_bf16 && !out_bf16)) return MU_ERR_BAD_ARGUMENT;
    cudaStream_t s = (cudaStream_t)stream;
    const dim3 grid(max_tiles, (n + mu::MOE_TN - 1) / mu::MOE_TN), block(256);
    typedef __nv_bfloat16 bf;
#define MU_MOE(T, TO, G)                                                                                             \
    return mu::launch_pdl(mu::moe_gemm_kernel<T, TO, G>, grid, block, 0, s, 1, (const T*)x, ldx, pair_of, top,        \
                          (const T*)w1, (const T*)w2, expert_stride, ldw, tile_info, n_tiles, n, k, (TO*)out, ldo, act)
    if (w2) {
        if (is_bf16 && out_bf16) MU_MOE(bf, bf, true);
        if (is_bf16) MU_MOE(bf, float, true);
        MU_MOE(float, float, true);
    }
    if (is_bf16 && out_bf16) MU_MOE(bf, bf, false);
    if (is_bf16) MU_MOE(bf, float, false);
    MU_MOE(float, float, false);
#undef MU_MOE
}

// x (the experts' input rows, bfloat16 if x_bf16 else float32) is needed when a pair may have no slot.
MU_EXPORT int mu_moe_combine(const float* y, long long ldy, const int* slot_of, const float* weight_of, int n_tokens,
                             int top, int width, float* out, long long ldo, void* stream, const void* x, long long ldx,
                             int x_bf16, const float* shared, long long lds, const float* shared_gate, int add) {
    if (n_tokens <= 0) return MU_OK;
    if (!y || !slot_of || !weight_of || !out || top <= 0 || width <= 0) return MU_ERR_BAD_ARGUMENT;
    const dim3 grid(n_tokens), block(width >= 1024 ? 256 : 128);
    const bool vec = width % 4 == 0 && ldy % 4 == 0 && ldo % 4 == 0 && ((uintptr_t)y & 15) == 0 && ((uintptr_t)out & 15) == 0 &&
                     (!x || (ldx % 4 == 0 && ((uintptr_t)x & (x_bf16 ? 7 : 15)) == 0)) &&
                     (!shared || (lds % 4 == 0 && ((uintptr_t)shared & 15) == 0));
    if (vec) {
        const dim3 vblock(width >= 1024 ? 256 : width >= 512 ? 128 : 64);
#define MU_COMBINE(TX, TOP)                                                                                            \
    return mu::launch_pdl(mu::moe_combine_vec_kernel<TX, TOP>, grid, vblock, 0, (cudaStream_t)stream, 1, y, ldy, slot_of, \
                          weight_of, top, width, out, ldo, (const TX*)x, ldx, shared, lds, shared_gate, add)
        if (x_bf16) {
            if (top == 2) MU_COMBINE(__nv_bfloat16, 2);
            if (top == 4) MU_COMBINE(__nv_bfloat16, 4);
            if (top == 6) MU_COMBINE(__nv_bfloat16, 6);
            if (top == 8) MU_COMBINE(__nv_bfloat16, 8);
            MU_COMBINE(__nv_bfloat16, 0);
        }
        if (top == 2) MU_COMBINE(float, 2);
        if (top == 4) MU_COMBINE(float, 4);
        if (top == 6) MU_COMBINE(float, 6);
        if (top == 8) MU_COMBINE(float, 8);
        MU_COMBINE(float, 0);
#undef MU_COMBINE
    }
    if (x_bf16)
        return mu::launch_pdl(mu::moe_combine_kernel<__nv_bfloat16>, grid, block, 0, (cudaStream_t)stream, 1, y, ldy,
                              slot_of, weight_of, top, width, out, ldo, (const __nv_bfloat16*)x, ldx, shared, lds,
                              shared_gate, add);
    return mu::launch_pdl(mu::moe_combine_kernel<float>, grid, block, 0, (cudaStream_t)stream, 1, y, ldy, slot_of,
                          weight_of, top, width, out, ldo, (const float*)x, ldx, shared, lds, shared_gate, add);
}
