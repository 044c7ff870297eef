// Small element-by-element kernels around products.
//
// mu_gated_act    out[t][f] = act(a[t][f]) * a[t][F + f]: the two halves of one product's output (gate | up) of a
//                 gated feed-forward; the activation in float32, storage in the compute dtype.
// mu_scaled_sum   y (+)= a * p + b * q, float32: two branches that join with a weight each.
// mu_cast_rows    float32 rows to bfloat16 rows.
// mu_xielu        out = f(a) element by element with two learned numbers (p, q) read from the device:
//                 z > 0: softplus(p) z^2 + z / 2;  z <= 0: (1/2 + softplus(q)) (exp(z) - 1 - z) + z / 2.
//                 Float32 arithmetic, storage in the compute dtype; out may be a.
#include "common.cuh"

#include <math.h>

namespace mu {

__device__ __forceinline__ float gate_act(float z, int act) {
    if (act == ACT_SILU) return z / (1.0f + expf(-z));
    return apply_act(z, act);
}

template <typename T>
__global__ void gated_act_kernel(const T* __restrict__ a, long long lda, T* __restrict__ out, long long ldo, int n_rows,
                                 int width, int act) {
    pdl_trigger();
    pdl_wait();
    const long long total = (long long)n_rows * width;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const long long r = i / width;
        const int c = (int)(i % width);
        const float g = to_float(a[r * lda + c]), u = to_float(a[r * lda + width + c]);
        out[r * ldo + c] = from_float<T>(gate_act(g, act) * u);
    }
}

// bfloat16 rows whose halves are whole, aligned 16-byte pieces: eight entries a thread.
__global__ void gated_act_vec_kernel(const __nv_bfloat16* __restrict__ a, long long lda, __nv_bfloat16* __restrict__ out,
                                     long long ldo, int n_rows, int width, int act) {
    pdl_trigger();
    pdl_wait();
    const int pieces = width / 8;
    const long long total = (long long)n_rows * pieces;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const long long r = i / pieces;
        const int c = (int)(i % pieces) * 8;
        const uint4 gr = *reinterpret_cast<const uint4*>(a + r * lda + c);
        const uint4 ur = *reinterpret_cast<const uint4*>(a + r * lda + width + c);
        const __nv_bfloat162* g2 = reinterpret_cast<const __nv_bfloat162*>(&gr);
        const __nv_bfloat162* u2 = reinterpret_cast<const __nv_bfloat162*>(&ur);
        uint4 packed;
        __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&packed);
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const float2 g = __bfloat1622float2(g2[k]), u = __bfloat1622float2(u2[k]);
            o2[k] = __floats2bfloat162_rn(gate_act(g.x, act) * u.x, gate_act(g.y, act) * u.y);
        }
        *reinterpret_cast<uint4*>(out + r * ldo + c) = packed;
    }
}

__device__ __forceinline__ float xielu_f(float z, float a_pos, float a_neg) {
    return z > 0.0f ? fmaf(a_pos * z, z, 0.5f * z) : fmaf(a_neg, expm1f(z) - z, 0.5f * z);
}

// The same for an output that is rounded to bfloat16: e^z - 1 - z by its series near zero (five terms, to -1/4,
// where the next one is 4e-7 of the sum) and by the fast exponential beyond, where the sum is 0.03 or more and the
// exponential's error 1e-7.  The exact form costs more arithmetic than the row's bytes take to move.
__device__ __forceinline__ float xielu_bf16_f(float z, float a_pos, float a_neg) {
    const float half = 0.5f * z;
    const float series = z * z * fmaf(z, fmaf(z, fmaf(z, fmaf(z, 1.0f / 720.0f, 1.0f / 120.0f), 1.0f / 24.0f), 1.0f / 6.0f), 0.5f);
    const float far = __expf(z) - 1.0f - z;
    return z > 0.0f ? fmaf(a_pos * z, z, half) : fmaf(a_neg, z > -0.25f ? series : far, half);
}

template <typename T>
__global__ void xielu_kernel(const T* a, long long lda, const float* __restrict__ pair, T* out, long long ldo,
                             int n_rows, int width) {
    pdl_trigger();
    pdl_wait();
    const float p = pair[0], q = pair[1];
    const float a_pos = fmaxf(p, 0.0f) + log1pf(expf(-fabsf(p)));
    const float a_neg = 0.5f + fmaxf(q, 0.0f) + log1pf(expf(-fabsf(q)));
    const long long total = (long long)n_rows * width;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const long long r = i / width;
        const int c = (int)(i % width);
        out[r * ldo + c] = from_float<T>(xielu_f(to_float(a[r * lda + c]), a_pos, a_neg));
    }
}

// bfloat16 rows of whole, aligned 16-byte pieces: eight entries a thread.
__global__ void xielu_vec_kernel(const __nv_bfloat16* a, long long lda, const float* __restrict__ pair,
                                 __nv_bfloat16* out, long long ldo, int n_rows, int width) {
    pdl_trigger();
    pdl_wait();
    const float p = pair[0], q = pair[1];
    const float a_pos = fmaxf(p, 0.0f) + log1pf(expf(-fabsf(p)));
    const float a_neg = 0.5f + fmaxf(q, 0.0f) + log1pf(expf(-fabsf(q)));
    const int pieces = width / 8;
    const long long total = (long long)n_rows * pieces;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const long long r = i / pieces;
        const int c = (int)(i % pieces) * 8;
        const uint4 raw = *reinterpret_cast<const uint4*>(a + r * lda + c);
        const __nv_bfloat162* z2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
        uint4 packed;
        __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&packed);
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const float2 z = __bfloat1622float2(z2[k]);
            o2[k] = __floats2bfloat162_rn(xielu_bf16_f(z.x, a_pos, a_neg), xielu_bf16_f(z.y, a_pos, a_neg));
        }
        *reinterpret_cast<uint4*>(out + r * ldo + c) = packed;
    }
}

template <bool ADD>
__global__ void scaled_sum_kernel(const float* __restrict__ p, long long ldp, float a, const float* __restrict__ q,
                                  long long ldq, float b, float* __restrict__ y, long long ldy, int n_rows, int width) {
    pdl_trigger();
    pdl_wait();
    const long long total = (long long)n_rows * width;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const long long r = i / width;
        const int c = (int)(i % width);
        float v = a * p[r * ldp + c] + b * q[r * ldq + c];
        if (ADD) v += y[r * ldy + c];
        y[r * ldy + c] = v;
    }
}

__global__ void cast_rows_kernel(const float* __restrict__ x, long long ldx, __nv_bfloat16* __restrict__ y, long long ldy,
                                 int n_rows, int width) {
    pdl_trigger();
    pdl_wait();
    const long long total = (long long)n_rows * width;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const long long r = i / width;
        const int c = (int)(i % width);
        y[r * ldy + c] = __float2bfloat16_rn(x[r * ldx + c]);
    }
}

inline unsigned blocks_for(long long total) {
    const long long b = (total + 255) / 256;
    return (unsigned)(b > 8192 ? 8192 : b);
}

}  // namespace mu

MU_EXPORT int mu_gated_act(const void* a, long long lda, void* out, long long ldo, int n_rows, int width, int act,
                           int is_bf16, void* stream) {
    if (n_rows <= 0 || width <= 0) return MU_OK;
    if (!a || !out || act < 0 || act > mu::ACT_SILU) return MU_ERR_BAD_ARGUMENT;
    cudaStream_t s = (cudaStream_t)stream;
    const dim3 grid(mu::blocks_for((long long)n_rows * width)), block(256);
    if (is_bf16 && width % 8 == 0 && lda % 8 == 0 && ldo % 8 == 0 && ((uintptr_t)a & 15) == 0 && ((uintptr_t)out & 15) == 0)
        return mu::launch_pdl(mu::gated_act_vec_kernel, dim3(mu::blocks_for((long long)n_rows * width / 8)), block, 0, s, 1,
                              (const __nv_bfloat16*)a, lda, (__nv_bfloat16*)out, ldo, n_rows, width, act);
    if (is_bf16)
        return mu::launch_pdl(mu::gated_act_kernel<__nv_bfloat16>, grid, block, 0, s, 1, (const __nv_bfloat16*)a, lda,
                              (__nv_bfloat16*)out, ldo, n_rows, width, act);
    return mu::launch_pdl(mu::gated_act_kernel<float>, grid, block, 0, s, 1, (const float*)a, lda, (float*)out, ldo, n_rows,
                          width, act);
}

MU_EXPORT int mu_scaled_sum(const float* p, long long ldp, float a, const float* q, long long ldq, float b, float* y,
                            long long ldy, int n_rows, int width, int add, void* stream) {
    if (n_rows <= 0 || width <= 0) return MU_OK;
    if (!p || !q || !y) return MU_ERR_BAD_ARGUMENT;
    cudaStream_t s = (cudaStream_t)stream;
    const dim3 grid(mu::blocks_for((long long)n_rows * width)), block(256);
    if (add) return mu::launch_pdl(mu::scaled_sum_kernel<true>, grid, block, 0, s, 1, p, ldp, a, q, ldq, b, y, ldy, n_rows, width);
    return mu::launch_pdl(mu::scaled_sum_kernel<false>, grid, block, 0, s, 1, p, ldp, a, q, ldq, b, y, ldy, n_rows, width);
}

MU_EXPORT int mu_cast_rows(const float* x, long long ldx, void* y, long long ldy, int n_rows, int width, void* stream) {
    if (n_rows <= 0 || width <= 0) return MU_OK;
    if (!x || !y) return MU_ERR_BAD_ARGUMENT;
    cudaStream_t s = (cudaStream_t)stream;
    const dim3 grid(mu::blocks_for((long long)n_rows * width)), block(256);
    return mu::launch_pdl(mu::cast_rows_kernel, grid, block, 0, s, 1, x, ldx, (__nv_bfloat16*)y, ldy, n_rows, width);
}

MU_EXPORT int mu_xielu(const void* a, long long lda, const float* pair, void* out, long long ldo, int n_rows, int width,
                       int is_bf16, void* stream) {
    if (n_rows <= 0 || width <= 0) return MU_OK;
    if (!a || !out || !pair) return MU_ERR_BAD_ARGUMENT;
    cudaStream_t s = (cudaStream_t)stream;
    const dim3 grid(mu::blocks_for((long long)n_rows * width)), block(256);
    if (is_bf16 && width % 8 == 0 && lda % 8 == 0 && ldo % 8 == 0 && ((uintptr_t)a & 15) == 0 && ((uintptr_t)out & 15) == 0)
        return mu::launch_pdl(mu::xielu_vec_kernel, dim3(mu::blocks_for((long long)n_rows * width / 8)), block, 0, s, 1,
                              (const __nv_bfloat16*)a, lda, pair, (__nv_bfloat16*)out, ldo, n_rows, width);
    if (is_bf16)
        return mu::launch_pdl(mu::xielu_kernel<__nv_bfloat16>, grid, block, 0, s, 1, (const __nv_bfloat16*)a, lda, pair,
                              (__nv_bfloat16*)out, ldo, n_rows, width);
    return mu::launch_pdl(mu::xielu_kernel<float>, grid, block, 0, s, 1, (const float*)a, lda, pair, (float*)out, ldo,
                          n_rows, width);
}
