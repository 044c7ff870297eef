// A state-space mixer with a matrix state per head (the state-space-duality form), token by token.
//
// Per sequence the mixer keeps, in float32, the last taps - 1 inputs of its short convolution and per head a
// state S [N][P]:
//     state[slot] = [ conv tail: (taps - 1) x channels, oldest first | S: heads x N x P ]
// mu_ssd_conv   out[t][c] = silu(bias[c] + sum_j w[c][j] in[t - taps + 1 + j][c]) over the step's tokens of
//               each sequence, the inputs before the step's first token taken from the tail (zeros when the
//               sequence starts: a slot's state is cleared when it is taken); float32 out.
//               When every sequence brings one token the same launch moves the tail on; otherwise
//               mu_ssd_conv_tail does, after it.
// mu_ssd_scan   per (sequence, head, a few columns of S), the step's tokens in order:
//               dt = softplus(dt_raw + dt_bias), S = exp(-exp(A_log) dt) S + dt B x^T, y = S^T C + D x;
//               everything float32; head h reads B and C of group h / (heads / groups).
// mu_gated_group_norm   y * silu(z), unit rms over each of `parts` equal parts of the row (eps inside the
//               root), times a weight; output in the compute dtype.  With `gate_after` the order is the other
//               one: y to unit rms per part, times the weight, times silu(z).
#include "common.cuh"

#include <math.h>

namespace mu {

__device__ __forceinline__ float silu_f(float z) { return z / (1.0f + expf(-z)); }
__device__ __forceinline__ float softplus_f(float z) { return fmaxf(z, 0.0f) + log1pf(expf(-fabsf(z))); }

// seq_first[s] .. seq_first[s + 1] - 1 are the flat tokens of the step's s-th sequence.
template <typename TE>
__global__ void ssd_conv_kernel(const TE* __restrict__ u, long long ldu, const float* __restrict__ weight,
                                const float* __restrict__ bias, int channels, int taps, int n_tokens,
                                const int* __restrict__ tok_seq, const int* __restrict__ seq_first,
                                const int* __restrict__ seq_slots, float* __restrict__ state, long long state_stride,
                                int move_tail, float* __restrict__ out) {
    pdl_trigger();
    pdl_wait();
    const int t = blockIdx.x, c = blockIdx.y * blockDim.x + threadIdx.x;
    if (c >= channels) return;
    const int s = tok_seq[t];
    const int first = seq_first[s];
    float* tail = state + (long long)seq_slots[s] * state_stride;
    float acc = bias ? bias[c] : 0.0f;
    for (int j = 0; j < taps; ++j) {
        const int li = t - first - (taps - 1) + j;                 // index within the step's tokens of this sequence
        const float x = li >= 0 ? to_float(u[(long long)(first + li) * ldu + c])
                                : tail[(long long)(taps - 1 + li) * channels + c];
        acc = fmaf(weight[(long long)c * taps + j], x, acc);
    }
    out[(long long)t * channels + c] = silu_f(acc);
    if (move_tail) {                                              // one token per sequence: this thread alone touches tail[.][c]
        for (int k = 0; k + 1 < taps - 1; ++k) tail[(long long)k * channels + c] = tail[(long long)(k + 1) * channels + c];
        if (taps > 1) tail[(long long)(taps - 2) * channels + c] = to_float(u[(long long)t * ldu + c]);
    }
}

template <typename TE>
__global__ void ssd_conv_tail_kernel(const TE* __restrict__ u, long long ldu, int channels, int taps, int n_seqs,
                                     const int* __restrict__ seq_first, const int* __restrict__ seq_slots,
                                     float* __restrict__ state, long long state_stride) {
    pdl_trigger();
    pdl_wait();
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (long long)n_seqs * channels) return;
    const int s = (int)(idx / channels), c = (int)(idx % channels);
    const int first = seq_first[s], count = seq_first[s + 1] - first;
    float* tail = state + (long long)seq_slots[s] * state_stride;
    // in ascending order: entry k takes what lay count entries later, which this thread has not written yet
    for (int k = 0; k < taps - 1; ++k) {
        const int li = count - (taps - 1) + k;
        tail[(long long)k * channels + c] = li >= 0 ? to_float(u[(long long)(first + li) * ldu + c])
                                                    : tail[(long long)(taps - 1 + li) * channels + c];
    }
}

// One block per (sequence, head); thread (p, part) owns the state entries S[n][p] with n = part, part + parts, ...
// in shared memory, so the update and the product with C need no exchange but the final sum over the parts.
template <typename TE>
__global__ void ssd_scan_kernel(const float* __restrict__ xbc, int channels, const TE* __restrict__ dt_raw, long long lddt,
                                const float* __restrict__ dt_bias, const float* __restrict__ a_log,
                                const float* __restrict__ skip, int n_heads, int P, int N, int groups, int parts,
                                const int* __restrict__ seq_first, const int* __restrict__ seq_slots,
                                float* __restrict__ state, long long state_stride, long long state_offset,
                                float* __restrict__ y) {
    extern __shared__ float smem[];
    float* S = smem;                       // [N][P]
    float* Bs = S + N * P;                 // [N]
    float* Cs = Bs + N;                    // [N]
    float* xs = Cs + N;                    // [P]
    float* red = xs + P;                   // [parts][P]
    pdl_trigger();
    pdl_wait();
    const int s = blockIdx.x, h = blockIdx.y, tid = threadIdx.x;
    const int p = tid % P, part = tid / P;
    const int g = h / (n_heads / groups);
    const int inner = n_heads * P;
    const int first = seq_first[s], count = seq_first[s + 1] - first;
    float* mine = state + (long long)seq_slots[s] * state_stride + state_offset + (long long)h * N * P;
    for (int e = tid; e < N * P; e += blockDim.x) S[e] = mine[e];
    const float rate = expf(a_log[h]), bias = dt_bias[h], d_skip = skip[h];
    __syncthreads();
    for (int li = 0; li < count; ++li) {
        const int t = first + li;
        const float* row = xbc + (long long)t * channels;
        for (int n = tid; n < N; n += blockDim.x) {
            Bs[n] = row[inner + g * N + n];
            Cs[n] = row[inner + groups * N + g * N + n];
        }
        for (int i = tid; i < P; i += blockDim.x) xs[i] = row[h * P + i];
        const float dt = softplus_f(to_float(dt_raw[(long long)t * lddt + h]) + bias);
        const float decay = expf(-rate * dt);
        __syncthreads();
        const float x = xs[p];
        float acc = 0.0f;
        for (int n = part; n < N; n += parts) {
            const float v = fmaf(decay, S[n * P + p], dt * Bs[n] * x);
            S[n * P + p] = v;
            acc = fmaf(v, Cs[n], acc);
        }
        red[part * P + p] = acc;
        __syncthreads();
        if (part == 0) {
            float sum = 0.0f;
            for (int k = 0; k < parts; ++k) sum += red[k * P + p];
            y[(long long)t * inner + h * P + p] = fmaf(d_skip, x, sum);
        }
    }
    __syncthreads();
    for (int e = tid; e < N * P; e += blockDim.x) mine[e] = S[e];
}

// The same recurrence with the state in registers: a block per (sequence, head, a few columns of S); LPC lanes own
// one column p, lane i of them the entries S[i NS .. i NS + NS - 1][p], so a step is NS fused multiply-adds for the
// update and NS for the product with C, with no barrier; the sums over a column's lanes are made 16 steps at a time.
// B, C, x, dt and the decay of 16 steps at a time come through shared memory in two stages (cp.async, 4 bytes a copy
// where 16 would not be aligned), the next 16 steps on their way while these are worked on.  N <= LPC * NS <= 128
// (larger states take the kernel above).
constexpr int SC_STEPS = 16;

__device__ __forceinline__ void cp_async16(void* dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src)
                 : "memory");
}
__device__ __forceinline__ void cp_async4(void* dst, const void* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src)
                 : "memory");
}

// One step of a lane's NS state entries: S = dec S + B dx, and the lane's share of S . C (two running sums, so that
// the additions of a step do not all wait for one another).
template <int NS>
__device__ __forceinline__ float scan_step(float (&S)[NS], const float* __restrict__ bp, const float* __restrict__ cp,
                                           float dx, float dec) {
    float sum0 = 0.0f, sum1 = 0.0f;
    if (NS % 4 == 0) {
#pragma unroll
        for (int i = 0; i < NS; i += 4) {
            const float4 b = *reinterpret_cast<const float4*>(bp + i);
            const float4 c = *reinterpret_cast<const float4*>(cp + i);
            S[i] = fmaf(dec, S[i], b.x * dx);
            S[i + 1] = fmaf(dec, S[i + 1], b.y * dx);
            S[i + 2] = fmaf(dec, S[i + 2], b.z * dx);
            S[i + 3] = fmaf(dec, S[i + 3], b.w * dx);
            sum0 = fmaf(S[i], c.x, sum0);
            sum1 = fmaf(S[i + 1], c.y, sum1);
            sum0 = fmaf(S[i + 2], c.z, sum0);
            sum1 = fmaf(S[i + 3], c.w, sum1);
        }
    } else {
#pragma unroll
        for (int i = 0; i < NS; ++i) {
            S[i] = fmaf(dec, S[i], bp[i] * dx);
            sum0 = fmaf(S[i], cp[i], sum0);
        }
    }
    return sum0 + sum1;
}

// LPC: lanes that share a column of S (16: a warp takes two columns; 32: one, which doubles the warps a step of a
// given size keeps busy).
template <typename TE, int NS, int LPC>
__global__ void __launch_bounds__(128)
ssd_scan_cols_kernel(const float* __restrict__ xbc, int channels, const TE* __restrict__ dt_raw, long long lddt,
                     const float* __restrict__ dt_bias, const float* __restrict__ a_log, const float* __restrict__ skip,
                     int n_heads, int P, int N, int groups, const int* __restrict__ seq_first,
                     const int* __restrict__ seq_slots, float* __restrict__ state, long long state_stride,
                     long long state_offset, float* __restrict__ y) {
    constexpr int NPAD = LPC * NS;
    constexpr int SC_COLS = 4 * (32 / LPC);                  // columns of a block: four warps
    __shared__ __align__(16) float Bs[2][SC_STEPS][NPAD], Cs[2][SC_STEPS][NPAD], xs[2][SC_STEPS][SC_COLS], dts[2][SC_STEPS],
        decs[2][SC_STEPS];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, part = lane % LPC;
    const int pl = warp * (32 / LPC) + lane / LPC;
    for (int i = tid; i < 2 * SC_STEPS * NPAD; i += blockDim.x) {
        (&Bs[0][0][0])[i] = 0.0f;
        (&Cs[0][0][0])[i] = 0.0f;
    }
    for (int i = tid; i < 2 * SC_STEPS * SC_COLS; i += blockDim.x) (&xs[0][0][0])[i] = 0.0f;
    pdl_trigger();
    pdl_wait();
    __syncthreads();
    const int s = blockIdx.x, h = blockIdx.y, col0 = blockIdx.z * SC_COLS;
    const int p = col0 + pl;
    const bool live = p < P;
    const int g = h / (n_heads / groups);
    const int inner = n_heads * P;
    const int first = seq_first[s], count = seq_first[s + 1] - first;
    float* mine = state + (long long)seq_slots[s] * state_stride + state_offset + (long long)h * N * P;
    float S[NS];
#pragma unroll
    for (int i = 0; i < NS; ++i) {
        const int n = part * NS + i;
        S[i] = (live && n < N) ? mine[(long long)n * P + p] : 0.0f;
    }
    const float rate = expf(a_log[h]), bias = dt_bias[h], d_skip = skip[h];
    const int n_chunks = (count + SC_STEPS - 1) / SC_STEPS;

    // 16-byte copies where every piece of a row starts on such a boundary, 4-byte copies otherwise
    const bool wide = channels % 4 == 0 && N % 4 == 0 && inner % 4 == 0 && ((uintptr_t)xbc & 15) == 0;
    const int b_at = inner + g * N, c_at = inner + groups * N + g * N;
    auto issue = [&](int chunk, int buf) {
        const int left = min(SC_STEPS, count - chunk * SC_STEPS);
        const float* base = xbc + (long long)(first + chunk * SC_STEPS) * channels;
        for (int tt = 0; tt < left; ++tt) {
            const float* row = base + (long long)tt * channels;
            if (wide) {
                for (int n = tid * 4; n < N; n += blockDim.x * 4) {
                    cp_async16(&Bs[buf][tt][n], row + b_at + n);
                    cp_async16(&Cs[buf][tt][n], row + c_at + n);
                }
            } else {
                for (int n = tid; n < N; n += blockDim.x) {
                    cp_async4(&Bs[buf][tt][n], row + b_at + n);
                    cp_async4(&Cs[buf][tt][n], row + c_at + n);
                }
            }
        }
        {
            const int tt = tid / SC_COLS, col = tid % SC_COLS;       // 16 steps x the block's columns
            if (tt < left && tt < SC_STEPS && col0 + col < P) cp_async4(&xs[buf][tt][col], base + (long long)tt * channels + h * P + col0 + col);
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    auto raw_dt = [&](int chunk) {
        const int li = chunk * SC_STEPS + tid;
        return (tid < SC_STEPS && li < count) ? to_float(dt_raw[(long long)(first + li) * lddt + h]) : 0.0f;
    };
    auto put_dt = [&](float raw, int buf) {
        if (tid < SC_STEPS) {
            const float dt = softplus_f(raw + bias);
            dts[buf][tid] = dt;
            decs[buf][tid] = expf(-rate * dt);
        }
    };
    if (n_chunks > 0) {
        issue(0, 0);
        put_dt(raw_dt(0), 0);
    }
    for (int c = 0; c < n_chunks; ++c) {
        const int buf = c & 1;
        float next_raw = 0.0f;
        if (c + 1 < n_chunks) {
            issue(c + 1, buf ^ 1);
            next_raw = raw_dt(c + 1);
            asm volatile("cp.async.wait_group 1;" ::: "memory");
        } else {
            asm volatile("cp.async.wait_group 0;" ::: "memory");
        }
        __syncthreads();
        const int left = min(SC_STEPS, count - c * SC_STEPS);
        // the 16 steps unrolled: a step's sum over the 16 lanes of a column is not made at once; each lane keeps its
        // partial sum of every step, and at the end the 16 x 16 partial sums are added crosswise in 15 shuffles, after
        // which lane i holds step i's sum.  So the only chain from step to step is the state's own.
        float acc[SC_STEPS];
        if (left == SC_STEPS) {                               // a whole chunk: no branch between the steps
#pragma unroll
            for (int tt = 0; tt < SC_STEPS; ++tt)
                acc[tt] = scan_step<NS>(S, &Bs[buf][tt][part * NS], &Cs[buf][tt][part * NS], dts[buf][tt] * xs[buf][tt][pl],
                                        decs[buf][tt]);
        } else {
#pragma unroll
            for (int tt = 0; tt < SC_STEPS; ++tt) {
                acc[tt] = 0.0f;
                if (tt < left)
                    acc[tt] = scan_step<NS>(S, &Bs[buf][tt][part * NS], &Cs[buf][tt][part * NS],
                                            dts[buf][tt] * xs[buf][tt][pl], decs[buf][tt]);
            }
        }
        if (LPC == 32) {
#pragma unroll
            for (int k = 0; k < SC_STEPS; ++k) acc[k] += __shfl_xor_sync(0xffffffffu, acc[k], 16);
        }
#pragma unroll
        for (int width = 8; width >= 1; width >>= 1) {
#pragma unroll
            for (int k = 0; k < width; ++k) {
                const bool upper = (part & width) != 0;
                const float send = upper ? acc[k] : acc[k + width];
                const float keep = upper ? acc[k + width] : acc[k];
                acc[k] = keep + __shfl_xor_sync(0xffffffffu, send, width);
            }
        }
        if (part < left && live)                              // (part < 16: with 32 lanes a column both halves hold the sums)
            y[(long long)(first + c * SC_STEPS + part) * inner + h * P + p] = fmaf(d_skip, xs[buf][part][pl], acc[0]);
        if (c + 1 < n_chunks) put_dt(next_raw, buf ^ 1);
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < NS; ++i) {
        const int n = part * NS + i;
        if (live && n < N) mine[(long long)n * P + p] = S[i];
    }
}

constexpr int GN_KEEP = 8;       // gated values a thread keeps between the statistics and the output

template <typename TE>
__global__ void __launch_bounds__(256)
gated_group_norm_kernel(const float* __restrict__ y, long long ldy, const TE* __restrict__ z, long long ldz,
                        const float* __restrict__ weight, int width, float eps, TE* __restrict__ out, long long ldo,
                        int gate_after) {
    __shared__ float scratch[32];
    pdl_trigger();
    pdl_wait();
    const int t = blockIdx.x, part = blockIdx.y;
    const float* ys = y + (long long)t * ldy + (long long)part * width;
    const TE* zs = z + (long long)t * ldz + (long long)part * width;
    float kept[GN_KEEP];
    float sq = 0.0f;
#pragma unroll
    for (int i = 0; i < GN_KEEP; ++i) {
        const int d = threadIdx.x + i * blockDim.x;
        kept[i] = d < width ? (gate_after ? ys[d] : ys[d] * silu_f(to_float(zs[d]))) : 0.0f;
        sq += kept[i] * kept[i];
    }
    for (int d = threadIdx.x + GN_KEEP * blockDim.x; d < width; d += blockDim.x) {
        const float v = gate_after ? ys[d] : ys[d] * silu_f(to_float(zs[d]));
        sq += v * v;
    }
    const float inv = 1.0f / sqrtf(block_sum(sq, scratch) / (float)width + eps);
    TE* dst = out + (long long)t * ldo + (long long)part * width;
    const float* w = weight + (long long)part * width;
#pragma unroll
    for (int i = 0; i < GN_KEEP; ++i) {
        const int d = threadIdx.x + i * blockDim.x;
        if (d < width) dst[d] = from_float<TE>(gate_after ? kept[i] * inv * w[d] * silu_f(to_float(zs[d])) : kept[i] * inv * w[d]);
    }
    for (int d = threadIdx.x + GN_KEEP * blockDim.x; d < width; d += blockDim.x)
        dst[d] = from_float<TE>(ys[d] * silu_f(to_float(zs[d])) * inv * w[d]);
}

// The same for parts of up to 32 * GN_KEEP entries (a head's values, as a rule): a warp a part, one or four parts a
// block, no barrier; the gate and the weight are on their way before the statistics are known.
template <typename TE>
__global__ void __launch_bounds__(128)
gated_group_norm_warp_kernel(const float* __restrict__ y, long long ldy, const TE* __restrict__ z, long long ldz,
                             const float* __restrict__ weight, int width, int parts, long long n_parts, float eps,
                             TE* __restrict__ out, long long ldo, int gate_after) {
    pdl_trigger();
    pdl_wait();
    const long long item = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (item >= n_parts) return;
    const int lane = threadIdx.x & 31;
    const long long t = item / parts;
    const int part = (int)(item % parts);
    const float* ys = y + t * ldy + (long long)part * width;
    const TE* zs = z + t * ldz + (long long)part * width;
    const float* w = weight + (long long)part * width;
    float kept[GN_KEEP], gate[GN_KEEP], wk[GN_KEEP];
    float sq = 0.0f;
#pragma unroll
    for (int i = 0; i < GN_KEEP; ++i) {
        const int d = lane + 32 * i;
        const bool in = d < width;
        gate[i] = in ? silu_f(to_float(zs[d])) : 0.0f;
        wk[i] = in ? w[d] : 0.0f;
        kept[i] = in ? (gate_after ? ys[d] : ys[d] * gate[i]) : 0.0f;
        sq = fmaf(kept[i], kept[i], sq);
    }
    const float inv = 1.0f / sqrtf(warp_sum(sq) / (float)width + eps);
    TE* dst = out + t * ldo + (long long)part * width;
#pragma unroll
    for (int i = 0; i < GN_KEEP; ++i) {
        const int d = lane + 32 * i;
        if (d < width) dst[d] = from_float<TE>(gate_after ? kept[i] * inv * wk[i] * gate[i] : kept[i] * inv * wk[i]);
    }
}

}  // namespace mu

// u: the convolution's input channels of the step's tokens ([T, channels] view of the projection, compute dtype).
// single_tokens: every sequence of the step brings exactly one token (the tail is moved on by the same launch).
MU_EXPORT int mu_ssd_conv(const void* u, long long ldu, int u_bf16, const float* weight, const float* bias, int channels,
                          int taps, int n_tokens, int n_seqs, const int* tok_seq, const int* seq_first,
                          const int* seq_slots, float* state, long long state_stride, int single_tokens, float* out,
                          void* stream) {
    if (n_tokens <= 0) return MU_OK;
    if (!u || !weight || !tok_seq || !seq_first || !seq_slots || !state || !out || channels <= 0 || taps < 1)
        return MU_ERR_BAD_ARGUMENT;
    cudaStream_t s = (cudaStream_t)stream;
    typedef __nv_bfloat16 bf;
    const dim3 grid(n_tokens, (channels + 255) / 256), block(256);
    int code = u_bf16 ? mu::launch_pdl(mu::ssd_conv_kernel<bf>, grid, block, 0, s, 1, (const bf*)u, ldu, weight, bias,
                                       channels, taps, n_tokens, tok_seq, seq_first, seq_slots, state, state_stride,
                                       single_tokens, out)
                      : mu::launch_pdl(mu::ssd_conv_kernel<float>, grid, block, 0, s, 1, (const float*)u, ldu, weight,
                                       bias, channels, taps, n_tokens, tok_seq, seq_first, seq_slots, state,
                                       state_stride, single_tokens, out);
    if (code != MU_OK || single_tokens || taps == 1) return code;
    const long long cells = (long long)n_seqs * channels;
    const dim3 tail_grid((unsigned)((cells + 255) / 256));
    return u_bf16 ? mu::launch_pdl(mu::ssd_conv_tail_kernel<bf>, tail_grid, block, 0, s, 1, (const bf*)u, ldu, channels,
                                   taps, n_seqs, seq_first, seq_slots, state, state_stride)
                  : mu::launch_pdl(mu::ssd_conv_tail_kernel<float>, tail_grid, block, 0, s, 1, (const float*)u, ldu,
                                   channels, taps, n_seqs, seq_first, seq_slots, state, state_stride);
}

MU_EXPORT int mu_ssd_scan(const float* xbc, int channels, const void* dt_raw, long long lddt, int dt_bf16,
                          const float* dt_bias, const float* a_log, const float* skip, int n_seqs, int n_heads, int P,
                          int N, int groups, const int* seq_first, const int* seq_slots, float* state,
                          long long state_stride, long long state_offset, float* y, int long_steps, void* stream) {
    if (n_seqs <= 0) return MU_OK;
    if (!xbc || !dt_raw || !dt_bias || !a_log || !skip || !seq_first || !seq_slots || !state || !y || n_heads <= 0 ||
        P <= 0 || N <= 0 || groups <= 0 || n_heads % groups)
        return MU_ERR_BAD_ARGUMENT;
    cudaStream_t s = (cudaStream_t)stream;
    typedef __nv_bfloat16 bf;
    if (N <= 128) {                                   // the state in registers, 8 columns of S a block
        const dim3 block(128);
#define MU_SCAN_COLS(NS, LPC)                                                                                          \
    do {                                                                                                               \
        const dim3 grid(n_seqs, n_heads, (P + 4 * (32 / LPC) - 1) / (4 * (32 / LPC)));                                 \
        return dt_bf16 ? mu::launch_pdl(mu::ssd_scan_cols_kernel<bf, NS, LPC>, grid, block, 0, s, 1, xbc, channels,    \
                                        (const bf*)dt_raw, lddt, dt_bias, a_log, skip, n_heads, P, N, groups,          \
                                        seq_first, seq_slots, state, state_stride, state_offset, y)                    \
                       : mu::launch_pdl(mu::ssd_scan_cols_kernel<float, NS, LPC>, grid, block, 0, s, 1, xbc, channels, \
                                        (const float*)dt_raw, lddt, dt_bias, a_log, skip, n_heads, P, N, groups,       \
                                        seq_first, seq_slots, state, state_stride, state_offset, y);                   \
    } while (0)
        if (N <= 16) MU_SCAN_COLS(1, 16);
        if (N <= 32) MU_SCAN_COLS(2, 16);
        if (N <= 64) MU_SCAN_COLS(4, 16);
        if (!long_steps) MU_SCAN_COLS(8, 16);         // a few tokens a sequence: fewer, larger blocks
        MU_SCAN_COLS(4, 32);                          // 65 .. 128 over many tokens: a warp a column, twice the warps
#undef MU_SCAN_COLS
    }
    if (P > 1024) return MU_ERR_UNSUPPORTED_SIZE;
    int parts = 256 / P;
    if (parts < 1) parts = 1;
    if (parts > N) parts = N;
    const size_t smem = ((size_t)N * P + 2 * (size_t)N + P + (size_t)parts * P) * sizeof(float);
    if (smem > 48 * 1024) {
        if (smem > 200 * 1024) return MU_ERR_UNSUPPORTED_SIZE;
        const void* fn = dt_bf16 ? (const void*)mu::ssd_scan_kernel<bf> : (const void*)mu::ssd_scan_kernel<float>;
        if (cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
            return MU_ERR_LAUNCH;
    }
    const dim3 grid(n_seqs, n_heads), block(P * parts);
    return dt_bf16 ? mu::launch_pdl(mu::ssd_scan_kernel<bf>, grid, block, smem, s, 1, xbc, channels, (const bf*)dt_raw, lddt,
                                    dt_bias, a_log, skip, n_heads, P, N, groups, parts, seq_first, seq_slots, state,
                                    state_stride, state_offset, y)
                   : mu::launch_pdl(mu::ssd_scan_kernel<float>, grid, block, smem, s, 1, xbc, channels,
                                    (const float*)dt_raw, lddt, dt_bias, a_log, skip, n_heads, P, N, groups, parts,
                                    seq_first, seq_slots, state, state_stride, state_offset, y);
}

MU_EXPORT int mu_gated_group_norm(const float* y, long long ldy, const void* z, long long ldz, const float* weight,
                                  int n_tokens, int inner, int parts, float eps, void* out, long long ldo, int is_bf16,
                                  void* stream, int gate_after) {
    if (n_tokens <= 0) return MU_OK;
    if (!y || !z || !weight || !out || inner <= 0 || parts <= 0 || inner % parts) return MU_ERR_BAD_ARGUMENT;
    cudaStream_t s = (cudaStream_t)stream;
    const int width = inner / parts;
    typedef __nv_bfloat16 bf;
    if (width <= 32 * mu::GN_KEEP && parts > 1) {
        const long long n_parts = (long long)n_tokens * parts;
        const int warps = n_parts >= 4096 ? 4 : 1;            // a few parts: a block each, spread over the SMs
        const dim3 grid((unsigned)((n_parts + warps - 1) / warps)), block(32 * warps);
        return is_bf16 ? mu::launch_pdl(mu::gated_group_norm_warp_kernel<bf>, grid, block, 0, s, 1, y, ldy, (const bf*)z,
                                        ldz, weight, width, parts, n_parts, eps, (bf*)out, ldo, gate_after)
                       : mu::launch_pdl(mu::gated_group_norm_warp_kernel<float>, grid, block, 0, s, 1, y, ldy,
                                        (const float*)z, ldz, weight, width, parts, n_parts, eps, (float*)out, ldo,
                                        gate_after);
    }
    const dim3 grid(n_tokens, parts), block(width >= 1024 ? 256 : 128);
    return is_bf16 ? mu::launch_pdl(mu::gated_group_norm_kernel<bf>, grid, block, 0, s, 1, y, ldy, (const bf*)z, ldz, weight,
                                    width, eps, (bf*)out, ldo, gate_after)
                   : mu::launch_pdl(mu::gated_group_norm_kernel<float>, grid, block, 0, s, 1, y, ldy, (const float*)z, ldz,
                                    weight, width, eps, (float*)out, ldo, gate_after);
}
