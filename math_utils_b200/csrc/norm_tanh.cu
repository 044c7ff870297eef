// Norms without a mean, and a sigmoid gate.
//
// dynamic_tanh:  y = tanh(alpha * x) * w + b          (no statistics of the row; alpha a scalar on the device)
//                with ADD the result is added to what y holds (a sublayer's normed output joining the
//                float32 residual stream); input always float32, output float32 or the compute dtype.
// rms_norm:      y = x / sqrt(mean(x^2) + eps) * w, statistics in float32.
// sigmoid_gate:  o *= 1 / (1 + exp(-g)), element by element, in float32.
// rms_norm_pair: two RMS norms of the same rows (one statistic, two weights, two outputs).
// softcap:       x <- cap * tanh(x / cap) on float32 rows, in place.
#include "common.cuh"

#include <math.h>

namespace mu {

template <typename TO, bool ADD>
__global__ void dynamic_tanh_kernel(const float* __restrict__ x, long long ldx, const int* __restrict__ rows,
                                    const float* __restrict__ w, const float* __restrict__ b,
                                    const float* __restrict__ alpha, TO* __restrict__ y, long long ldy, int hidden) {
    pdl_trigger();
    pdl_wait();
    const int r = blockIdx.x;
    const float a = alpha[0];
    const float* src = x + (rows ? (long long)rows[r] : (long long)r) * ldx;
    TO* dst = y + (long long)r * ldy;
    for (int d = blockIdx.y * blockDim.x + threadIdx.x; d < hidden; d += gridDim.y * blockDim.x) {
        float v = tanhf(a * src[d]) * w[d] + (b ? b[d] : 0.0f);
        if (ADD) v += to_float(dst[d]);
        dst[d] = from_float<TO>(v);
    }
}

template <typename TI, typename TO>
__global__ void rms_norm_kernel(const TI* __restrict__ x, long long ldx, const float* __restrict__ w,
                                TO* __restrict__ y, long long ldy, int n, float eps) {
    __shared__ float scratch[32];
    pdl_trigger();
    pdl_wait();
    const TI* src = x + (long long)blockIdx.x * ldx;
    TO* dst = y + (long long)blockIdx.x * ldy;
    float s = 0.0f;
    for (int d = threadIdx.x; d < n; d += blockDim.x) {
        const float v = to_float(src[d]);
        s += v * v;
    }
    const float inv = 1.0f / sqrtf(block_sum(s, scratch) / (float)n + eps);
    for (int d = threadIdx.x; d < n; d += blockDim.x) dst[d] = from_float<TO>(to_float(src[d]) * inv * w[d]);
}

// y (+)= scale * v / sqrt(mean(v^2) + eps) * (offset + w) for float32 rows v = x (optionally the rows that `rows`
// picks), or v = a * x + b * x2 (two branches that join with a weight each, summed on the way in): a norm on a
// sublayer's output that joins the residual stream with a multiplier, or a norm whose weight is stored around zero
// (offset 1).  `copy` (optional, bfloat16) receives what y then holds: the next sublayer's input in the compute
// dtype, without a pass of its own.
template <typename TO, bool ADD>
__global__ void rms_norm_out_kernel(const float* __restrict__ x, long long ldx, const float* __restrict__ x2, long long ldx2,
                                    float a, float b, const int* __restrict__ rows, const float* __restrict__ w,
                                    float offset, float scale, float eps, TO* __restrict__ y, long long ldy,
                                    __nv_bfloat16* __restrict__ copy, long long ldc, int n) {
    __shared__ float scratch[32];
    pdl_trigger();
    pdl_wait();
    const int r = blockIdx.x;
    const long long from = rows ? (long long)rows[r] : (long long)r;
    const float* src = x + from * ldx;
    const float* src2 = x2 ? x2 + from * ldx2 : nullptr;
    TO* dst = y + (long long)r * ldy;
    float s = 0.0f;
    for (int d = threadIdx.x; d < n; d += blockDim.x) {
        const float v = src2 ? a * src[d] + b * src2[d] : src[d];
        s += v * v;
    }
    const float inv = 1.0f / sqrtf(block_sum(s, scratch) / (float)n + eps);
    for (int d = threadIdx.x; d < n; d += blockDim.x) {
        float v = (src2 ? a * src[d] + b * src2[d] : src[d]) * inv * (offset + w[d]) * scale;
        if (ADD) v += to_float(dst[d]);
        dst[d] = from_float<TO>(v);
        if (copy) copy[(long long)r * ldc + d] = __float2bfloat16_rn(v);
    }
}

// The same for rows of up to 4,096 values that are whole, aligned 16-byte pieces: a block of 256 threads reads its
// row once, four values a load, and keeps it in registers between the statistics and the output.
template <typename TO, bool ADD>
__global__ void __launch_bounds__(256)
rms_norm_out_vec_kernel(const float* __restrict__ x, long long ldx, const float* __restrict__ x2, long long ldx2,
                        float a, float b, const int* __restrict__ rows, const float* __restrict__ w, float offset,
                        float scale, float eps, TO* __restrict__ y, long long ldy, __nv_bfloat16* __restrict__ copy,
                        long long ldc, int n) {
    __shared__ float scratch[32];
    pdl_trigger();
    pdl_wait();
    const int r = blockIdx.x, n4 = n / 4;
    const long long from = rows ? (long long)rows[r] : (long long)r;
    const float4* src = reinterpret_cast<const float4*>(x + from * ldx);
    const float4* src2 = x2 ? reinterpret_cast<const float4*>(x2 + from * ldx2) : nullptr;
    float4 v[4];
    float s = 0.0f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int idx = threadIdx.x + 256 * i;
        v[i] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        if (idx < n4) {
            v[i] = src[idx];
            if (src2) {
                const float4 u = src2[idx];
                v[i] = make_float4(a * v[i].x + b * u.x, a * v[i].y + b * u.y, a * v[i].z + b * u.z, a * v[i].w + b * u.w);
            }
        }
        s += (v[i].x * v[i].x + v[i].y * v[i].y) + (v[i].z * v[i].z + v[i].w * v[i].w);
    }
    const float inv = scale / sqrtf(block_sum(s, scratch) / (float)n + eps);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int idx = threadIdx.x + 256 * i;
        if (idx < n4) {
            const float4 g = reinterpret_cast<const float4*>(w)[idx];
            float4 o = make_float4(v[i].x * inv * (offset + g.x), v[i].y * inv * (offset + g.y),
                                   v[i].z * inv * (offset + g.z), v[i].w * inv * (offset + g.w));
            if (ADD) {
                const float4 old = reinterpret_cast<const float4*>(y + (long long)r * ldy)[idx];
                o.x += old.x; o.y += old.y; o.z += old.z; o.w += old.w;
            }
            if (sizeof(TO) == 4) {
                reinterpret_cast<float4*>(y + (long long)r * ldy)[idx] = o;
            } else {
                __nv_bfloat162 lo = __floats2bfloat162_rn(o.x, o.y), hi = __floats2bfloat162_rn(o.z, o.w);
                uint2 packed;
                packed.x = *reinterpret_cast<uint32_t*>(&lo);
                packed.y = *reinterpret_cast<uint32_t*>(&hi);
                reinterpret_cast<uint2*>(y + (long long)r * ldy)[idx] = packed;
            }
            if (copy) {
                __nv_bfloat162 lo = __floats2bfloat162_rn(o.x, o.y), hi = __floats2bfloat162_rn(o.z, o.w);
                uint2 packed;
                packed.x = *reinterpret_cast<uint32_t*>(&lo);
                packed.y = *reinterpret_cast<uint32_t*>(&hi);
                reinterpret_cast<uint2*>(copy + (long long)r * ldc)[idx] = packed;
            }
        }
    }
}

template <typename T>
__global__ void sigmoid_gate_kernel(T* __restrict__ o, long long ldo, const T* __restrict__ g, long long ldg,
                                    int n_rows, int width) {
    pdl_trigger();
    pdl_wait();
    const long long total = (long long)n_rows * width;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (long long)gridDim.x * blockDim.x) {
        const long long r = i / width;
        const int c = (int)(i % width);
        const float z = to_float(g[r * ldg + c]);
        const float v = to_float(o[r * ldo + c]) / (1.0f + expf(-z));
        o[r * ldo + c] = from_float<T>(v);
    }
}

// Two RMS norms of the same rows with the same eps: one pass over x, one statistic, two weights, two outputs.
template <typename TO>
__global__ void __launch_bounds__(256)
rms_norm_pair_kernel(const float* __restrict__ x, long long ldx, const float* __restrict__ w1,
                     const float* __restrict__ w2, float eps, TO* __restrict__ y1, long long ldy1,
                     TO* __restrict__ y2, long long ldy2, int n, int vec) {
    __shared__ float scratch[32];
    pdl_trigger();
    pdl_wait();
    const int r = blockIdx.x;
    const float* src = x + (long long)r * ldx;
    float s = 0.0f;
    if (vec) {
        // up to 4096 entries: a thread keeps its four float4 between the two passes
        const float4* src4 = reinterpret_cast<const float4*>(src);
        const int n4 = n / 4;
        float4 v[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int idx = threadIdx.x + 256 * i;
            v[i] = idx < n4 ? src4[idx] : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            s += (v[i].x * v[i].x + v[i].y * v[i].y) + (v[i].z * v[i].z + v[i].w * v[i].w);
        }
        const float inv = 1.0f / sqrtf(block_sum(s, scratch) / (float)n + eps);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int idx = threadIdx.x + 256 * i;
            if (idx >= n4) continue;
            const float4 a = reinterpret_cast<const float4*>(w1)[idx], b = reinterpret_cast<const float4*>(w2)[idx];
            const float4 u = make_float4(v[i].x * inv, v[i].y * inv, v[i].z * inv, v[i].w * inv);
            const float4 o1 = make_float4(u.x * a.x, u.y * a.y, u.z * a.z, u.w * a.w);
            const float4 o2 = make_float4(u.x * b.x, u.y * b.y, u.z * b.z, u.w * b.w);
            if (sizeof(TO) == 4) {
                reinterpret_cast<float4*>(y1 + (long long)r * ldy1)[idx] = o1;
                reinterpret_cast<float4*>(y2 + (long long)r * ldy2)[idx] = o2;
            } else {
                __nv_bfloat162 p0 = __floats2bfloat162_rn(o1.x, o1.y), p1 = __floats2bfloat162_rn(o1.z, o1.w);
                __nv_bfloat162 q0 = __floats2bfloat162_rn(o2.x, o2.y), q1 = __floats2bfloat162_rn(o2.z, o2.w);
                uint2 pa, pb;
                pa.x = *reinterpret_cast<uint32_t*>(&p0); pa.y = *reinterpret_cast<uint32_t*>(&p1);
                pb.x = *reinterpret_cast<uint32_t*>(&q0); pb.y = *reinterpret_cast<uint32_t*>(&q1);
                reinterpret_cast<uint2*>(y1 + (long long)r * ldy1)[idx] = pa;
                reinterpret_cast<uint2*>(y2 + (long long)r * ldy2)[idx] = pb;
            }
        }
        return;
    }
    for (int d = threadIdx.x; d < n; d += blockDim.x) s += src[d] * src[d];
    const float inv = 1.0f / sqrtf(block_sum(s, scratch) / (float)n + eps);
    for (int d = threadIdx.x; d < n; d += blockDim.x) {
        const float u = src[d] * inv;
        y1[(long long)r * ldy1 + d] = from_float<TO>(u * w1[d]);
        y2[(long long)r * ldy2 + d] = from_float<TO>(u * w2[d]);
    }
}

// x <- cap * tanh(x / cap), float32 rows in place.
__global__ void softcap_kernel(float* __restrict__ x, long long ldx, int n_rows, int width, float cap) {
    pdl_trigger();
    pdl_wait();
    const long long total = (long long)n_rows * width;
    const float inv = 1.0f / cap;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (long long)gridDim.x * blockDim.x) {
        const long long r = i / width;
        const int c = (int)(i % width);
        x[r * ldx + c] = cap * tanhf(x[r * ldx + c] * inv);
    }
}

}  // namespace mu

// y (+)= tanh(alpha x) w + b for n_rows rows (optionally the rows that `rows` picks from x).
// out_bf16: y is bfloat16 (else float32); add: accumulate into y (float32 only).
MU_EXPORT int mu_dynamic_tanh(const float* x, long long ldx, const int* rows, const float* w, const float* b,
                              const float* alpha, void* y, long long ldy, int n_rows, int hidden, int out_bf16,
                              int add, void* stream) {
    if (n_rows <= 0) return MU_OK;
    if (hidden <= 0 || !x || !w || !alpha || !y || (add && out_bf16)) return MU_ERR_BAD_ARGUMENT;
    cudaStream_t s = (cudaStream_t)stream;
    // few rows (single-token steps): several blocks share a row, so that the tanh of a row is spread over the SMs
    const int threads = hidden >= 1024 ? 256 : 128;
    const int per_row = n_rows >= 256 ? 1 : (hidden + 2 * threads - 1) / (2 * threads);
    const dim3 grid(n_rows, per_row > 0 ? per_row : 1), block(threads);
    if (out_bf16)
        return mu::launch_pdl(mu::dynamic_tanh_kernel<__nv_bfloat16, false>, grid, block, 0, s, 1, x, ldx, rows, w, b,
                              alpha, (__nv_bfloat16*)y, ldy, hidden);
    if (add)
        return mu::launch_pdl(mu::dynamic_tanh_kernel<float, true>, grid, block, 0, s, 1, x, ldx, rows, w, b, alpha,
                              (float*)y, ldy, hidden);
    return mu::launch_pdl(mu::dynamic_tanh_kernel<float, false>, grid, block, 0, s, 1, x, ldx, rows, w, b, alpha,
                          (float*)y, ldy, hidden);
}

// y = rms_norm(x) * w over rows of n values; x and y are bfloat16 or float32 as the flags say.
MU_EXPORT int mu_rms_norm(const void* x, long long ldx, int x_bf16, const float* w, void* y, long long ldy,
                          int y_bf16, int n_rows, int n, float eps, void* stream) {
    if (n_rows <= 0) return MU_OK;
    if (n <= 0 || !x || !w || !y) return MU_ERR_BAD_ARGUMENT;
    cudaStream_t s = (cudaStream_t)stream;
    const dim3 grid(n_rows), block(n >= 1024 ? 256 : 128);
    typedef __nv_bfloat16 bf;
    if (x_bf16 && y_bf16)
        return mu::launch_pdl(mu::rms_norm_kernel<bf, bf>, grid, block, 0, s, 1, (const bf*)x, ldx, w, (bf*)y, ldy, n, eps);
    if (x_bf16)
        return mu::launch_pdl(mu::rms_norm_kernel<bf, float>, grid, block, 0, s, 1, (const bf*)x, ldx, w, (float*)y, ldy, n, eps);
    if (y_bf16)
        return mu::launch_pdl(mu::rms_norm_kernel<float, bf>, grid, block, 0, s, 1, (const float*)x, ldx, w, (bf*)y, ldy, n, eps);
    return mu::launch_pdl(mu::rms_norm_kernel<float, float>, grid, block, 0, s, 1, (const float*)x, ldx, w, (float*)y, ldy, n, eps);
}

// y (+)= scale * rms_norm(v) * (offset + w) with v = x, or a * x + b * x2 when x2 is given; x, x2 float32, y float32
// or bfloat16 (add: float32 only).
MU_EXPORT int mu_rms_norm_out(const float* x, long long ldx, const float* x2, long long ldx2, float a, float b,
                              const int* rows, const float* w, float offset, float scale, float eps, void* y,
                              long long ldy, int y_bf16, int add, void* copy, long long ldc, int n_rows, int n,
                              void* stream) {
    if (n_rows <= 0) return MU_OK;
    if (n <= 0 || !x || !w || !y || (add && y_bf16)) return MU_ERR_BAD_ARGUMENT;
    cudaStream_t s = (cudaStream_t)stream;
    typedef __nv_bfloat16 bf;
    const bool vec = n % 4 == 0 && n <= 4096 && ldx % 4 == 0 && ((uintptr_t)x & 15) == 0 && ((uintptr_t)w & 15) == 0 &&
                     (!x2 || (ldx2 % 4 == 0 && ((uintptr_t)x2 & 15) == 0)) && ldy % 4 == 0 &&
                     ((uintptr_t)y & 15) == 0 && (!copy || (ldc % 4 == 0 && ((uintptr_t)copy & 7) == 0));
    const dim3 grid(n_rows), block(vec ? 256 : (n >= 1024 ? 256 : 128));
#define MU_RMS_OUT(KERNEL, TO, ADD)                                                                                    \
    return mu::launch_pdl(mu::KERNEL<TO, ADD>, grid, block, 0, s, 1, x, ldx, x2, ldx2, a, b, rows, w, offset, scale,   \
                          eps, (TO*)y, ldy, (bf*)copy, ldc, n)
    if (vec) {
        if (y_bf16) MU_RMS_OUT(rms_norm_out_vec_kernel, bf, false);
        if (add) MU_RMS_OUT(rms_norm_out_vec_kernel, float, true);
        MU_RMS_OUT(rms_norm_out_vec_kernel, float, false);
    }
    if (y_bf16) MU_RMS_OUT(rms_norm_out_kernel, bf, false);
    if (add) MU_RMS_OUT(rms_norm_out_kernel, float, true);
    MU_RMS_OUT(rms_norm_out_kernel, float, false);
#undef MU_RMS_OUT
}

// o[r, c] *= sigmoid(g[r, c]).
MU_EXPORT int mu_sigmoid_gate(void* o, long long ldo, const void* g, long long ldg, int n_rows, int width, int is_bf16,
                              void* stream) {
    if (n_rows <= 0 || width <= 0) return MU_OK;
    if (!o || !g) return MU_ERR_BAD_ARGUMENT;
    cudaStream_t s = (cudaStream_t)stream;
    const long long total = (long long)n_rows * width;
    const dim3 grid((unsigned)((total + 255) / 256 > 4096 ? 4096 : (total + 255) / 256)), block(256);
    if (is_bf16)
        return mu::launch_pdl(mu::sigmoid_gate_kernel<__nv_bfloat16>, grid, block, 0, s, 1, (__nv_bfloat16*)o, ldo,
                              (const __nv_bfloat16*)g, ldg, n_rows, width);
    return mu::launch_pdl(mu::sigmoid_gate_kernel<float>, grid, block, 0, s, 1, (float*)o, ldo, (const float*)g, ldg,
                          n_rows, width);
}

// y1 = rms_norm(x) * w1 and y2 = rms_norm(x) * w2 (same eps) of float32 rows; both outputs float32 or both bfloat16.
MU_EXPORT int mu_rms_norm_pair(const float* x, long long ldx, const float* w1, const float* w2, float eps, void* y1,
                               long long ldy1, void* y2, long long ldy2, int y_bf16, int n_rows, int n, void* stream) {
    if (n_rows <= 0) return MU_OK;
    if (n <= 0 || !x || !w1 || !w2 || !y1 || !y2) return MU_ERR_BAD_ARGUMENT;
    cudaStream_t s = (cudaStream_t)stream;
    const int vec = n % 4 == 0 && n <= 4096 && ldx % 4 == 0 && ldy1 % 4 == 0 && ldy2 % 4 == 0 && ((uintptr_t)x & 15) == 0 &&
                    ((uintptr_t)w1 & 15) == 0 && ((uintptr_t)w2 & 15) == 0 && ((uintptr_t)y1 & 15) == 0 &&
                    ((uintptr_t)y2 & 15) == 0;
    const dim3 grid(n_rows), block(256);
    if (y_bf16)
        return mu::launch_pdl(mu::rms_norm_pair_kernel<__nv_bfloat16>, grid, block, 0, s, 1, x, ldx, w1, w2, eps,
                              (__nv_bfloat16*)y1, ldy1, (__nv_bfloat16*)y2, ldy2, n, vec);
    return mu::launch_pdl(mu::rms_norm_pair_kernel<float>, grid, block, 0, s, 1, x, ldx, w1, w2, eps, (float*)y1, ldy1,
                          (float*)y2, ldy2, n, vec);
}

// x <- cap * tanh(x / cap) on float32 rows, in place.
MU_EXPORT int mu_softcap(float* x, long long ldx, int n_rows, int width, float cap, void* stream) {
    if (n_rows <= 0 || width <= 0) return MU_OK;
    if (!x || !(cap > 0.0f)) return MU_ERR_BAD_ARGUMENT;
    const long long total = (long long)n_rows * width;
    const dim3 grid((unsigned)((total + 255) / 256 > 4096 ? 4096 : (total + 255) / 256)), block(256);
    return mu::launch_pdl(mu::softcap_kernel, grid, block, 0, (cudaStream_t)stream, 1, x, ldx, n_rows, width, cap);
}
