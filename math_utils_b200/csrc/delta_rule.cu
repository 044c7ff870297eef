// The gated delta rule: a recurrent mixer with a matrix state S [dk][dv] per head, token by token.
//
// Per sequence the mixer keeps, in float32,
//     state[slot] = [ conv tail: (taps - 1) x channels, oldest first | S: heads x dv x dk ]
// (a head's S is stored column after column: the dk entries that one value entry reads lie together).  The short
// convolution with silu is mu_ssd_conv's; its float32 output row is [ q: kv heads x dk | k: kv heads x dk |
// v: heads x dv ].  Head h reads the queries and keys of kv head h / (heads / kv_heads).
//
// mu_delta_prepare   per token: every kv head's q and k become unit vectors, x / sqrt(sum x^2 + 1e-6), q also times
//                    q_scale, in place; kq = q . k of the finished vectors; per head beta = sigmoid(b_raw) and
//                    decay = exp(-exp(A_log) * softplus(a_raw + dt_bias)).  Everything float32.
// mu_delta_scan      per (sequence, head, 16 columns of S), the step's tokens in order:
//                        S <- decay S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q
//                    A column of S (one value entry) lives in the registers of 8 lanes; the two sums a token needs
//                    (S^T k and S^T q of the decayed state) are made together, and the read-out of the written
//                    state follows as S^T q + u (k . q), so a token costs one exchange between the lanes, not two.
//                    q, k, v, beta, decay and k . q of 16 tokens at a time go through shared memory.
//                    The order of every sum is fixed by the column alone: a token's result does not depend on how
//                    the sequence was cut into steps or on the batch.
#include "common.cuh"

#include <math.h>

namespace mu {

__device__ __forceinline__ float dl_softplus(float z) { return fmaxf(z, 0.0f) + log1pf(expf(-fabsf(z))); }

template <typename TE>
__global__ void __launch_bounds__(128)
delta_prepare_kernel(float* __restrict__ qkv, int channels, const TE* __restrict__ b_raw, long long ldb,
                     const TE* __restrict__ a_raw, long long lda, const float* __restrict__ a_log,
                     const float* __restrict__ dt_bias, int n_heads, int n_kv_heads, int dk, float q_scale,
                     float* __restrict__ kq, float* __restrict__ beta, float* __restrict__ decay) {
    pdl_trigger();
    pdl_wait();
    const int t = blockIdx.x, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, warps = blockDim.x >> 5;
    float* row = qkv + (long long)t * channels;
    for (int g = warp; g < n_kv_heads; g += warps) {
        float* qv = row + (long long)g * dk;
        float* kv = row + (long long)(n_kv_heads + g) * dk;
        float sq = 0.0f, sk = 0.0f;
        for (int d = lane; d < dk; d += 32) {
            sq = fmaf(qv[d], qv[d], sq);
            sk = fmaf(kv[d], kv[d], sk);
        }
        const float iq = q_scale / sqrtf(warp_sum(sq) + 1e-6f), ik = 1.0f / sqrtf(warp_sum(sk) + 1e-6f);
        float dot = 0.0f;
        for (int d = lane; d < dk; d += 32) {
            const float a = qv[d] * iq, b = kv[d] * ik;
            qv[d] = a;
            kv[d] = b;
            dot = fmaf(a, b, dot);
        }
        dot = warp_sum(dot);
        if (lane == 0) kq[(long long)t * n_kv_heads + g] = dot;
    }
    for (int h = tid; h < n_heads; h += blockDim.x) {
        const float b = to_float(b_raw[(long long)t * ldb + h]);
        const float a = to_float(a_raw[(long long)t * lda + h]);
        beta[(long long)t * n_heads + h] = 1.0f / (1.0f + expf(-b));
        decay[(long long)t * n_heads + h] = expf(-expf(a_log[h]) * dl_softplus(a + dt_bias[h]));
    }
}

constexpr int DL_LANES = 8;       // lanes that share a column of S
constexpr int DL_COLS = 16;       // columns a block takes
constexpr int DL_CHUNK = 16;      // tokens staged at a time

// R: entries of a column a lane holds; dk <= DL_LANES * R.  Lane l holds entries l * R .. l * R + R - 1.
template <int R>
__global__ void __launch_bounds__(DL_LANES * DL_COLS)
delta_scan_kernel(const float* __restrict__ qkv, int channels, const float* __restrict__ kq,
                  const float* __restrict__ beta, const float* __restrict__ decay, int n_heads, int n_kv_heads, int dk,
                  int dv, const int* __restrict__ seq_first, const int* __restrict__ seq_slots,
                  float* __restrict__ state, long long state_stride, long long state_offset, float* __restrict__ out) {
    constexpr int DKP = DL_LANES * R;
    __shared__ __align__(16) float ks[DL_CHUNK][DKP];
    __shared__ __align__(16) float qs[DL_CHUNK][DKP];
    __shared__ float vs[DL_CHUNK][DL_COLS];
    __shared__ float sc[DL_CHUNK][4];                        // beta, decay, k . q
    pdl_trigger();
    pdl_wait();
    const int s = blockIdx.x, h = blockIdx.y, col0 = blockIdx.z * DL_COLS;
    const int tid = threadIdx.x, c = tid / DL_LANES, l = tid % DL_LANES;
    const int g = h / (n_heads / n_kv_heads);
    const int j = col0 + c;
    const bool live = j < dv;
    const int first = seq_first[s], count = seq_first[s + 1] - first;
    float* mine = state + (long long)seq_slots[s] * state_stride + state_offset + ((long long)h * dv + j) * dk;
    float S[R];
#pragma unroll
    for (int r = 0; r < R; ++r) {
        const int d = l * R + r;
        S[r] = live && d < dk ? mine[d] : 0.0f;
    }
    const long long q_off = (long long)g * dk, k_off = (long long)(n_kv_heads + g) * dk;
    const long long v_off = (long long)2 * n_kv_heads * dk + (long long)h * dv + col0;
    for (int li0 = 0; li0 < count; li0 += DL_CHUNK) {
        const int n = min(DL_CHUNK, count - li0);
        __syncthreads();                                     // the chunk before is done with
        for (int i = tid; i < n * DKP; i += blockDim.x) {
            const int tok = i / DKP, d = i % DKP;
            const float* row = qkv + (long long)(first + li0 + tok) * channels;
            ks[tok][d] = d < dk ? row[k_off + d] : 0.0f;
            qs[tok][d] = d < dk ? row[q_off + d] : 0.0f;
        }
        for (int i = tid; i < n * DL_COLS; i += blockDim.x) {
            const int tok = i / DL_COLS, cc = i % DL_COLS;
            vs[tok][cc] = col0 + cc < dv ? qkv[(long long)(first + li0 + tok) * channels + v_off + cc] : 0.0f;
        }
        for (int tok = tid; tok < n; tok += blockDim.x) {
            const long long t = first + li0 + tok;
            sc[tok][0] = beta[t * n_heads + h];
            sc[tok][1] = decay[t * n_heads + h];
            sc[tok][2] = kq[t * n_kv_heads + g];
        }
        __syncthreads();
        for (int tok = 0; tok < n; ++tok) {
            const float b = sc[tok][0], a = sc[tok][1], qk = sc[tok][2];
            float kr[R];
            float d1 = 0.0f, d2 = 0.0f;
#pragma unroll
            for (int r = 0; r < R; ++r) {
                kr[r] = ks[tok][l * R + r];
                S[r] *= a;
                d1 = fmaf(S[r], kr[r], d1);
                d2 = fmaf(S[r], qs[tok][l * R + r], d2);
            }
#pragma unroll
            for (int o = DL_LANES / 2; o > 0; o >>= 1) {
                d1 += __shfl_xor_sync(0xffffffffu, d1, o);
                d2 += __shfl_xor_sync(0xffffffffu, d2, o);
            }
            const float u = b * (vs[tok][c] - d1);
#pragma unroll
            for (int r = 0; r < R; ++r) S[r] = fmaf(kr[r], u, S[r]);
            if (l == 0 && live)
                out[(long long)(first + li0 + tok) * n_heads * dv + (long long)h * dv + j] = fmaf(u, qk, d2);
        }
    }
#pragma unroll
    for (int r = 0; r < R; ++r) {
        const int d = l * R + r;
        if (live && d < dk) mine[d] = S[r];
    }
}

}  // namespace mu

// qkv: the convolution's float32 output rows [T][channels], channels = 2 * kv_heads * dk + heads * dv; q and k are
// finished in place.  b_raw, a_raw: [T][heads] views of the projection in the compute dtype.
MU_EXPORT int mu_delta_prepare(float* qkv, int channels, const void* b_raw, long long ldb, const void* a_raw,
                               long long lda, const float* a_log, const float* dt_bias, int n_tokens, int n_heads,
                               int n_kv_heads, int dk, float q_scale, float* kq, float* beta, float* decay,
                               int is_bf16, void* stream) {
    if (n_tokens <= 0) return MU_OK;
    if (!qkv || !b_raw || !a_raw || !a_log || !dt_bias || !kq || !beta || !decay || n_heads <= 0 || n_kv_heads <= 0 ||
        n_heads % n_kv_heads || dk <= 0 || channels < 2 * n_kv_heads * dk)
        return MU_ERR_BAD_ARGUMENT;
    cudaStream_t s = (cudaStream_t)stream;
    const dim3 grid(n_tokens), block(128);
    typedef __nv_bfloat16 bf;
    if (is_bf16)
        return mu::launch_pdl(mu::delta_prepare_kernel<bf>, grid, block, 0, s, 1, qkv, channels, (const bf*)b_raw, ldb,
                              (const bf*)a_raw, lda, a_log, dt_bias, n_heads, n_kv_heads, dk, q_scale, kq, beta, decay);
    return mu::launch_pdl(mu::delta_prepare_kernel<float>, grid, block, 0, s, 1, qkv, channels, (const float*)b_raw, ldb,
                          (const float*)a_raw, lda, a_log, dt_bias, n_heads, n_kv_heads, dk, q_scale, kq, beta, decay);
}

// The largest key size the scan takes.
MU_EXPORT int mu_delta_scan_max_dk() { return mu::DL_LANES * 32; }

MU_EXPORT int mu_delta_scan(const float* qkv, int channels, const float* kq, const float* beta, const float* decay,
                            int n_seqs, int n_heads, int n_kv_heads, int dk, int dv, const int* seq_first,
                            const int* seq_slots, float* state, long long state_stride, long long state_offset,
                            float* out, void* stream) {
    if (n_seqs <= 0) return MU_OK;
    if (!qkv || !kq || !beta || !decay || !seq_first || !seq_slots || !state || !out || n_heads <= 0 ||
        n_kv_heads <= 0 || n_heads % n_kv_heads || dk <= 0 || dv <= 0 ||
        channels != 2 * n_kv_heads * dk + n_heads * dv)
        return MU_ERR_BAD_ARGUMENT;
    if (dk > mu::DL_LANES * 32) return MU_ERR_UNSUPPORTED_SIZE;
    cudaStream_t s = (cudaStream_t)stream;
    const dim3 grid(n_seqs, n_heads, (dv + mu::DL_COLS - 1) / mu::DL_COLS), block(mu::DL_LANES * mu::DL_COLS);
#define MU_DELTA_SCAN(R)                                                                                              \
    return mu::launch_pdl(mu::delta_scan_kernel<R>, grid, block, 0, s, 1, qkv, channels, kq, beta, decay, n_heads,    \
                          n_kv_heads, dk, dv, seq_first, seq_slots, state, state_stride, state_offset, out)
    const int per = (dk + mu::DL_LANES - 1) / mu::DL_LANES;
    if (per <= 4) MU_DELTA_SCAN(4);
    if (per <= 8) MU_DELTA_SCAN(8);
    if (per <= 16) MU_DELTA_SCAN(16);
    MU_DELTA_SCAN(32);
#undef MU_DELTA_SCAN
}
