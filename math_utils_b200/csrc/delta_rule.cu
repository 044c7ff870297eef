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
//                    A column of S (one value entry) lives in the registers of 8 lanes.  The two sums a token needs
//                    are made together and of the state as the token found it: (decay S)^T k = decay (S^T k), and
//                    the read-out of the written state is decay (S^T q) + u (k . q).  So a token costs one exchange
//                    between the lanes, not two, and the decay is off the path that waits for it.
//                    q, k, v, beta, decay and k . q of 16 tokens at a time are copied to shared memory
//                    asynchronously, the next 16 while these are worked on.
//                    The order of every sum is fixed by the column alone: a token's result does not depend on how
//                    the sequence was cut into steps or on the batch.
#include "common.cuh"

#include <math.h>
#include <stdint.h>

#include <mutex>
#include <unordered_set>

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

constexpr int DL_COLS = 16;       // columns a block takes
constexpr int DL_CHUNK = 16;      // tokens staged at a time
constexpr int DL_MAX_DK = 256;    // the longest column

// Asynchronous copies global -> shared of 4 or 16 bytes, grouped and waited for by the issuing thread.
__device__ __forceinline__ void dl_copy4(float* dst, const float* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"((unsigned)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void dl_copy16(float* dst, const float* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((unsigned)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void dl_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void dl_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// Floats of one staged chunk: keys and queries padded to DKP entries, the block's values, (beta, decay, k . q, -).
__host__ __device__ constexpr int dl_chunk_floats(int dkp) { return DL_CHUNK * (2 * dkp + DL_COLS + 4); }

// LANES: lanes that share a column of S; R: entries of the column a lane holds (a multiple of 4); dk <= LANES * R.
// The column is dealt to the lanes four entries at a time: lane l holds entries 4 (l + LANES i) .. 4 (l + LANES i) + 3,
// i < R / 4, so that 8 neighbouring lanes read 128 consecutive bytes of a staged key at once.  (Measured at dk = 128:
// 8 lanes with 16 entries each beat 16 lanes with 8 and one more exchange.)  LANES and R follow from dk alone, so the
// order of the sums does too.
// VEC: dk, dv, the row length and the state's offset and stride are all multiples of 4, so keys, queries, values and
// the state move 16 bytes at a time.
template <int R, int LANES, bool VEC>
__global__ void __launch_bounds__(LANES * DL_COLS)
delta_scan_kernel(const float* __restrict__ qkv, int channels, const float* __restrict__ kq,
                  const float* __restrict__ beta, const float* __restrict__ decay, int n_heads, int n_kv_heads, int dk,
                  int dv, const int* __restrict__ seq_first, const int* __restrict__ seq_slots,
                  float* __restrict__ state, long long state_stride, long long state_offset, float* __restrict__ out) {
    constexpr int DL_LANES = LANES, DL_THREADS = LANES * DL_COLS;
    constexpr int DKP = DL_LANES * R, Q = R / 4, BUF = dl_chunk_floats(DKP);
    extern __shared__ __align__(16) float dl_smem[];
    const int s = blockIdx.x, h = blockIdx.y, col0 = blockIdx.z * DL_COLS;
    const int tid = threadIdx.x, c = tid / DL_LANES, l = tid % DL_LANES;
    const int g = h / (n_heads / n_kv_heads);
    const int j = col0 + c;
    const bool live = j < dv;
    for (int i = tid; i < 2 * BUF; i += DL_THREADS) dl_smem[i] = 0.0f;   // the padding past dk and dv stays zero
    pdl_wait();
    const int first = seq_first[s], count = seq_first[s + 1] - first;
    float* mine = state + (long long)seq_slots[s] * state_stride + state_offset + ((long long)h * dv + j) * dk;
    float S[R];
#pragma unroll
    for (int i = 0; i < Q; ++i) {
        const int d = 4 * (l + DL_LANES * i);
        if (VEC) {
            const float4 x = live && d < dk ? *reinterpret_cast<const float4*>(mine + d) : make_float4(0.f, 0.f, 0.f, 0.f);
            S[4 * i] = x.x, S[4 * i + 1] = x.y, S[4 * i + 2] = x.z, S[4 * i + 3] = x.w;
        } else {
#pragma unroll
            for (int e = 0; e < 4; ++e) S[4 * i + e] = live && d + e < dk ? mine[d + e] : 0.0f;
        }
    }
    const long long q_off = (long long)g * dk, k_off = (long long)(n_kv_heads + g) * dk;
    const long long v_off = (long long)2 * n_kv_heads * dk + (long long)h * dv + col0;
    // stages the chunk that starts at the sequence's li0-th token of this step into buffer `b`
    auto stage = [&](int li0, int b) {
        float* ks = dl_smem + b * BUF;
        float* qs = ks + DL_CHUNK * DKP;
        float* vs = qs + DL_CHUNK * DKP;
        float* sc = vs + DL_CHUNK * DL_COLS;
        const int n = min(DL_CHUNK, count - li0);
        if (VEC) {
            const int per = dk / 4;
            for (int i = tid; i < n * per; i += DL_THREADS) {
                const int tok = i / per, d = 4 * (i % per);
                const float* row = qkv + (long long)(first + li0 + tok) * channels;
                dl_copy16(ks + tok * DKP + d, row + k_off + d);
                dl_copy16(qs + tok * DKP + d, row + q_off + d);
            }
            for (int i = tid; i < n * (DL_COLS / 4); i += DL_THREADS) {
                const int tok = i / (DL_COLS / 4), cc = 4 * (i % (DL_COLS / 4));
                if (col0 + cc < dv)
                    dl_copy16(vs + tok * DL_COLS + cc, qkv + (long long)(first + li0 + tok) * channels + v_off + cc);
            }
        } else {
            for (int i = tid; i < n * dk; i += DL_THREADS) {
                const int tok = i / dk, d = i % dk;
                const float* row = qkv + (long long)(first + li0 + tok) * channels;
                dl_copy4(ks + tok * DKP + d, row + k_off + d);
                dl_copy4(qs + tok * DKP + d, row + q_off + d);
            }
            for (int i = tid; i < n * DL_COLS; i += DL_THREADS) {
                const int tok = i / DL_COLS, cc = i % DL_COLS;
                if (col0 + cc < dv)
                    dl_copy4(vs + tok * DL_COLS + cc, qkv + (long long)(first + li0 + tok) * channels + v_off + cc);
            }
        }
        for (int tok = tid; tok < n; tok += DL_THREADS) {
            const long long t = first + li0 + tok;
            dl_copy4(sc + tok * 4 + 0, beta + t * n_heads + h);
            dl_copy4(sc + tok * 4 + 1, decay + t * n_heads + h);
            dl_copy4(sc + tok * 4 + 2, kq + t * n_kv_heads + g);
        }
        dl_commit();
    };
    __syncthreads();                                         // the zeros are down before the first copies land
    if (count > 0) stage(0, 0);
    int b = 0;
    for (int li0 = 0; li0 < count; li0 += DL_CHUNK, b ^= 1) {
        const int n = min(DL_CHUNK, count - li0);
        if (li0 + DL_CHUNK < count) {
            stage(li0 + DL_CHUNK, b ^ 1);                    // the next chunk is on its way while this one is worked on
            dl_wait<1>();
        } else {
            dl_wait<0>();
        }
        __syncthreads();
        const float* ks = dl_smem + b * BUF;
        const float* qs = ks + DL_CHUNK * DKP;
        const float* vs = qs + DL_CHUNK * DKP;
        const float* sc = vs + DL_CHUNK * DL_COLS;
        // A token's keys, queries, value and scalars are read into registers while the token before it is still
        // waiting for its sums to come round the lanes.
        float4 kr[Q], qr[Q];
        float4 par = *reinterpret_cast<const float4*>(sc);                           // beta, decay, k . q
        float v = vs[c];
#pragma unroll
        for (int i = 0; i < Q; ++i) {
            kr[i] = *reinterpret_cast<const float4*>(ks + 4 * (l + DL_LANES * i));
            qr[i] = *reinterpret_cast<const float4*>(qs + 4 * (l + DL_LANES * i));
        }
        for (int tok = 0; tok < n; ++tok) {
            float d1[4] = {0.0f, 0.0f, 0.0f, 0.0f}, d2[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
            for (int i = 0; i < Q; ++i) {
                d1[0] = fmaf(S[4 * i], kr[i].x, d1[0]), d2[0] = fmaf(S[4 * i], qr[i].x, d2[0]);
                d1[1] = fmaf(S[4 * i + 1], kr[i].y, d1[1]), d2[1] = fmaf(S[4 * i + 1], qr[i].y, d2[1]);
                d1[2] = fmaf(S[4 * i + 2], kr[i].z, d1[2]), d2[2] = fmaf(S[4 * i + 2], qr[i].z, d2[2]);
                d1[3] = fmaf(S[4 * i + 3], kr[i].w, d1[3]), d2[3] = fmaf(S[4 * i + 3], qr[i].w, d2[3]);
            }
            float sk = (d1[0] + d1[1]) + (d1[2] + d1[3]), sq = (d2[0] + d2[1]) + (d2[2] + d2[3]);
            const int nxt = min(tok + 1, DL_CHUNK - 1);                              // the last one reads itself again
            float4 nk[Q];
#pragma unroll
            for (int i = 0; i < Q; ++i) {
                nk[i] = *reinterpret_cast<const float4*>(ks + nxt * DKP + 4 * (l + DL_LANES * i));
                qr[i] = *reinterpret_cast<const float4*>(qs + nxt * DKP + 4 * (l + DL_LANES * i));
            }
            const float4 npar = *reinterpret_cast<const float4*>(sc + nxt * 4);
            const float nv = vs[nxt * DL_COLS + c];
#pragma unroll
            for (int o = DL_LANES / 2; o > 0; o >>= 1) {
                sk += __shfl_xor_sync(0xffffffffu, sk, o);
                sq += __shfl_xor_sync(0xffffffffu, sq, o);
            }
            // the sums are of the state before its decay: (decay S)^T k = decay (S^T k)
            const float u = par.x * (v - par.y * sk);
#pragma unroll
            for (int i = 0; i < Q; ++i) {
                S[4 * i] = fmaf(kr[i].x, u, par.y * S[4 * i]);
                S[4 * i + 1] = fmaf(kr[i].y, u, par.y * S[4 * i + 1]);
                S[4 * i + 2] = fmaf(kr[i].z, u, par.y * S[4 * i + 2]);
                S[4 * i + 3] = fmaf(kr[i].w, u, par.y * S[4 * i + 3]);
                kr[i] = nk[i];
            }
            if (l == 0 && live)
                out[(long long)(first + li0 + tok) * n_heads * dv + (long long)h * dv + j] = fmaf(u, par.z, par.y * sq);
            par = npar;
            v = nv;
        }
        __syncthreads();                                     // this buffer is free for the chunk after the next
    }
    // Only now may the next kernel start: its blocks would wait beside this one's for the whole scan, and a block
    // here has one warp a scheduler, which every waiting warp there slows down.
    pdl_trigger();
#pragma unroll
    for (int i = 0; i < Q; ++i) {
        const int d = 4 * (l + DL_LANES * i);
        if (VEC) {
            if (live && d < dk)
                *reinterpret_cast<float4*>(mine + d) = make_float4(S[4 * i], S[4 * i + 1], S[4 * i + 2], S[4 * i + 3]);
        } else {
#pragma unroll
            for (int e = 0; e < 4; ++e)
                if (live && d + e < dk) mine[d + e] = S[4 * i + e];
        }
    }
}

// A kernel whose two buffers pass the default limit of dynamic shared memory asks for more, once.
inline bool dl_allow_shared(const void* kernel, size_t bytes) {
    static std::mutex mutex;
    static std::unordered_set<const void*> seen;
    if (bytes <= 48 * 1024) return true;
    std::lock_guard<std::mutex> lock(mutex);
    if (seen.count(kernel)) return true;
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes) != cudaSuccess) {
        cudaGetLastError();
        return false;
    }
    seen.insert(kernel);
    return true;
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
MU_EXPORT int mu_delta_scan_max_dk() { return mu::DL_MAX_DK; }

MU_EXPORT int mu_delta_scan(const float* qkv, int channels, const float* kq, const float* beta, const float* decay,
                            int n_seqs, int n_heads, int n_kv_heads, int dk, int dv, const int* seq_first,
                            const int* seq_slots, float* state, long long state_stride, long long state_offset,
                            float* out, int long_steps, void* stream) {
    if (n_seqs <= 0) return MU_OK;
    if (!qkv || !kq || !beta || !decay || !seq_first || !seq_slots || !state || !out || n_heads <= 0 ||
        n_kv_heads <= 0 || n_heads % n_kv_heads || dk <= 0 || dv <= 0 ||
        channels != 2 * n_kv_heads * dk + n_heads * dv)
        return MU_ERR_BAD_ARGUMENT;
    if (dk > mu::DL_MAX_DK) return MU_ERR_UNSUPPORTED_SIZE;
    cudaStream_t s = (cudaStream_t)stream;
    const dim3 grid(n_seqs, n_heads, (dv + mu::DL_COLS - 1) / mu::DL_COLS);
    const bool vec = dk % 4 == 0 && dv % 4 == 0 && channels % 4 == 0 && state_stride % 4 == 0 && state_offset % 4 == 0 &&
                     (reinterpret_cast<uintptr_t>(qkv) | reinterpret_cast<uintptr_t>(state)) % 16 == 0;
    // long_steps: many tokens a sequence (a prompt step).  The blocks then run for a long time with one warp a
    // scheduler; they start in plain stream order, on an empty device.
    // the two staging buffers of a block are most of what it needs of an SM: with the largest share of the on-chip
    // memory as shared memory several blocks fit, and the state is read once, so the L1 is no loss
#define MU_DELTA_SCAN_V(R, LANES, V)                                                                                  \
    do {                                                                                                              \
        const size_t smem = 2 * sizeof(float) * mu::dl_chunk_floats(LANES * R);                                       \
        const void* kernel = (const void*)mu::delta_scan_kernel<R, LANES, V>;                                         \
        if (!mu::dl_allow_shared(kernel, smem)) return MU_ERR_LAUNCH;                                                 \
        mu::prefer_shared_memory(kernel);                                                                             \
        if (long_steps)                                                                                               \
            return mu::launch_after(mu::delta_scan_kernel<R, LANES, V>, grid, dim3(LANES * mu::DL_COLS), smem, s, qkv, \
                                    channels, kq, beta, decay, n_heads, n_kv_heads, dk, dv, seq_first, seq_slots,     \
                                    state, state_stride, state_offset, out);                                          \
        return mu::launch_pdl(mu::delta_scan_kernel<R, LANES, V>, grid, dim3(LANES * mu::DL_COLS), smem, s, 1, qkv,   \
                              channels, kq, beta, decay, n_heads, n_kv_heads, dk, dv, seq_first, seq_slots, state,    \
                              state_stride, state_offset, out);                                                       \
    } while (0)
#define MU_DELTA_SCAN(R, LANES)                                                                                       \
    do {                                                                                                              \
        if (vec) MU_DELTA_SCAN_V(R, LANES, true);                                                                     \
        MU_DELTA_SCAN_V(R, LANES, false);                                                                             \
    } while (0)
    if (dk <= 32) MU_DELTA_SCAN(4, 8);
    if (dk <= 64) MU_DELTA_SCAN(8, 8);
    if (dk <= 128) MU_DELTA_SCAN(16, 8);
    MU_DELTA_SCAN(32, 8);
#undef MU_DELTA_SCAN_V
#undef MU_DELTA_SCAN
}
