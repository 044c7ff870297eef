// The experts' products on tensor cores (mma.sync m16n8k16, bfloat16, float32 accumulation).
//
// Same work list as the CUDA-core kernel of moe.cu: tiles of up to 32 or 64 slots of one expert (tile_info), rows of x
// gathered through the slots' pairs or taken by slot.  A block computes 32 or 64 rows x 128 output columns with eight
// warps, operands staged in shared memory by cp.async in chunks of 64 along k (two stages) and
// read as fragments with ldmatrix.  GATED: two weight stacks, out = silu(W1 x) * (W2 x).  Every output is one
// running sum over k in order, whatever shares its tile.
//
// The same kernel serves products PER HEAD (mu_heads_gemm): out[t, h, :] = W[h] x[t, h, :] for every token t and head
// h, the head taking the expert's place: tile (blockIdx.x, head blockIdx.z) covers tokens 32 blockIdx.x .. + 32, and
// a head's slice of x and of out starts x_group_offset / out_group_offset elements after the head before.
#include "common.cuh"

#include <math.h>

namespace mu {

constexpr int MM_COLS = 128, MM_THREADS = 256;
#ifndef MU_MM_K
#define MU_MM_K 64
#endif
#ifndef MU_MM_STAGES
#define MU_MM_STAGES 2
#endif
constexpr int MM_K = MU_MM_K, MM_STAGES = MU_MM_STAGES, MM_PITCH = MM_K + 8;

__device__ __forceinline__ void mm_mma(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void mm_ldmatrix_x4(uint32_t (&r)[4], const void* smem) {
    const uint32_t addr = (uint32_t)__cvta_generic_to_shared(smem);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
// 16 bytes to shared memory, of which the first `bytes` come from global memory and the rest are zero
__device__ __forceinline__ void mm_cp_async16(void* smem, const void* gmem, int bytes) {
    const uint32_t addr = (uint32_t)__cvta_generic_to_shared(smem);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" :: "r"(addr), "l"(gmem), "r"(bytes) : "memory");
}

// WM: row groups of 32.  WM = 1: 32 rows a block, a warp 32 x 16; WM = 2: 64 rows, a warp 32 x 32 (two warps along the
// rows, four along the columns): twice the arithmetic per fragment load, for experts that have the rows.
template <typename TO, bool GATED, int WM>
__global__ void __launch_bounds__(MM_THREADS)
moe_gemm_mma_kernel(const __nv_bfloat16* __restrict__ x, long long ldx, const int* __restrict__ pair_of, int top,
                    const __nv_bfloat16* __restrict__ w1, const __nv_bfloat16* __restrict__ w2, long long expert_stride,
                    long long ldw, const int* __restrict__ tile_info, const int* __restrict__ n_tiles, int n, int k,
                    TO* __restrict__ out, long long ldo, int n_rows, long long x_group_offset,
                    long long out_group_offset, const __nv_bfloat16* __restrict__ gate, long long ldg, int act) {
    extern __shared__ __align__(16) unsigned char mm_raw[];
    constexpr int MM_ROWS = 32 * WM, NW = 2 * WM;                               // rows a block; 8-column tiles a warp
    constexpr int STAGE = (MM_ROWS + (GATED ? 2 : 1) * MM_COLS) * MM_PITCH;      // elements per stage
    __nv_bfloat16* sm = reinterpret_cast<__nv_bfloat16*>(mm_raw);
    __shared__ int src_row[64];
    pdl_trigger();
    pdl_wait();
    const int tile = blockIdx.x;
    int e, slot0, rows;
    if (tile_info) {
        if (tile >= n_tiles[0]) return;
        e = tile_info[3 * tile], slot0 = tile_info[3 * tile + 1], rows = tile_info[3 * tile + 2];
    } else {                                                     // every group (head) has all n_rows rows
        e = blockIdx.z, slot0 = tile * MM_ROWS, rows = min(MM_ROWS, n_rows - slot0);
        if (rows <= 0) return;
    }
    x += (long long)e * x_group_offset;
    out += (long long)e * out_group_offset;
    if (gate) gate += (long long)e * out_group_offset;          // the gate lies as the output does
    const int n0 = blockIdx.y * MM_COLS;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    if (tid < MM_ROWS) {
        const int r = min(tid, rows - 1);                        // rows past the tile's end repeat its last row
        src_row[tid] = pair_of ? pair_of[slot0 + r] / top : slot0 + r;
    }
    __syncthreads();
    const __nv_bfloat16* w1e = w1 + (long long)e * expert_stride;
    const __nv_bfloat16* w2e = GATED ? w2 + (long long)e * expert_stride : nullptr;

    auto load = [&](int k0, int stage) {
        __nv_bfloat16* sa = sm + stage * STAGE;
        __nv_bfloat16* sb1 = sa + MM_ROWS * MM_PITCH;
        __nv_bfloat16* sb2 = sb1 + MM_COLS * MM_PITCH;
        constexpr int CPR = MM_K / 8;                            // 16-byte pieces a row
#pragma unroll
        for (int idx = tid; idx < MM_ROWS * CPR; idx += MM_THREADS) {
            const int r = idx / CPR, c = (idx % CPR) * 8;
            const int left = (k - (k0 + c)) * 2;
            const int bytes = left >= 16 ? 16 : (left > 0 ? left : 0);
            mm_cp_async16(sa + r * MM_PITCH + c, x + (long long)src_row[r] * ldx + (bytes ? k0 + c : 0), bytes);
        }
#pragma unroll
        for (int idx = tid; idx < MM_COLS * CPR; idx += MM_THREADS) {
            const int r = idx / CPR, c = (idx % CPR) * 8;
            const int left = (k - (k0 + c)) * 2;
            const int bytes = left >= 16 ? 16 : (left > 0 ? left : 0);
            const long long row = min(n0 + r, n - 1);            // columns past n repeat the last one
            mm_cp_async16(sb1 + r * MM_PITCH + c, w1e + row * ldw + (bytes ? k0 + c : 0), bytes);
            if (GATED) mm_cp_async16(sb2 + r * MM_PITCH + c, w2e + row * ldw + (bytes ? k0 + c : 0), bytes);
        }
    };

    float acc1[2][NW][4] = {}, acc2[GATED ? 2 : 1][NW][4] = {};
    const int row_base = WM == 2 ? (warp >> 2) * 32 : 0, col_base = WM == 2 ? (warp & 3) * 32 : warp * 16;
    const int chunks = (k + MM_K - 1) / MM_K;
    // a ring of MM_STAGES stages: MM_STAGES - 1 chunks on their way while one is worked on; a group is committed
    // for every chunk index, empty past the end, so that the wait below always counts the same
#pragma unroll
    for (int i = 0; i < MM_STAGES - 1; ++i) {
        if (i < chunks) load(i * MM_K, i);
        asm volatile("cp.async.commit_group;" ::: "memory");
    }
    for (int ch = 0; ch < chunks; ++ch) {
        const int stage = ch % MM_STAGES;
        asm volatile("cp.async.wait_group %0;" :: "n"(MM_STAGES - 2) : "memory");
        __syncthreads();                                         // chunk ch has landed; everyone is done with chunk ch - 1
        if (ch + MM_STAGES - 1 < chunks) load((ch + MM_STAGES - 1) * MM_K, (ch + MM_STAGES - 1) % MM_STAGES);
        asm volatile("cp.async.commit_group;" ::: "memory");
        const __nv_bfloat16* sa = sm + stage * STAGE;
        const __nv_bfloat16* sb1 = sa + MM_ROWS * MM_PITCH;
        const __nv_bfloat16* sb2 = sb1 + MM_COLS * MM_PITCH;
        const int brow = col_base + (lane & 7) + (lane >> 4) * 8, bcol = ((lane >> 3) & 1) * 8;
#pragma unroll
        for (int kk = 0; kk < MM_K; kk += 16) {
            uint32_t a[2][4], b[4];
            mm_ldmatrix_x4(a[0], sa + (row_base + (lane & 15)) * MM_PITCH + kk + (lane >> 4) * 8);
            mm_ldmatrix_x4(a[1], sa + (row_base + 16 + (lane & 15)) * MM_PITCH + kk + (lane >> 4) * 8);
#pragma unroll
            for (int j = 0; j < NW; j += 2) {
                mm_ldmatrix_x4(b, sb1 + (brow + 8 * j) * MM_PITCH + kk + bcol);
#pragma unroll
                for (int m = 0; m < 2; ++m) {
                    mm_mma(acc1[m][j], a[m], b[0], b[1]);
                    mm_mma(acc1[m][j + 1], a[m], b[2], b[3]);
                }
                if (GATED) {
                    mm_ldmatrix_x4(b, sb2 + (brow + 8 * j) * MM_PITCH + kk + bcol);
#pragma unroll
                    for (int m = 0; m < 2; ++m) {
                        mm_mma(acc2[m][j], a[m], b[0], b[1]);
                        mm_mma(acc2[m][j + 1], a[m], b[2], b[3]);
                    }
                }
            }
        }
    }
    const int g = lane >> 2, t4 = lane & 3;
#pragma unroll
    for (int m = 0; m < 2; ++m)
#pragma unroll
        for (int j = 0; j < NW; ++j)
#pragma unroll
            for (int half = 0; half < 2; ++half) {
                const int r = row_base + m * 16 + g + half * 8;
                const int col = n0 + col_base + j * 8 + 2 * t4;
                if (r >= rows || col >= n) continue;
                float v0 = acc1[m][j][2 * half], v1 = acc1[m][j][2 * half + 1];
                if (GATED) {
                    v0 = v0 / (1.0f + expf(-v0)) * acc2[m][j][2 * half];
                    v1 = v1 / (1.0f + expf(-v1)) * acc2[m][j][2 * half + 1];
                } else if (act == ACT_RELU2) {
                    v0 = relu2(v0);
                    v1 = relu2(v1);
                }
                if (gate) {                                      // out *= sigmoid(gate), in float32
                    const __nv_bfloat16* gp = gate + (long long)(slot0 + r) * ldg + col;
                    v0 = v0 / (1.0f + expf(-__bfloat162float(gp[0])));
                    if (col + 1 < n) v1 = v1 / (1.0f + expf(-__bfloat162float(gp[1])));
                }
                TO* dst = out + (long long)(slot0 + r) * ldo + col;
                dst[0] = from_float<TO>(v0);
                if (col + 1 < n) dst[1] = from_float<TO>(v1);
            }
}

template <typename TO, bool GATED, int WM>
int launch_moe_mma(dim3 grid, cudaStream_t s, const __nv_bfloat16* x, long long ldx, const int* pair_of, int top,
                   const __nv_bfloat16* w1, const __nv_bfloat16* w2, long long expert_stride, long long ldw,
                   const int* tile_info, const int* n_tiles, int n, int k, TO* out, long long ldo, int n_rows = 0,
                   long long x_group_offset = 0, long long out_group_offset = 0, const __nv_bfloat16* gate = nullptr,
                   long long ldg = 0, int act = 0) {
    constexpr size_t smem = MM_STAGES * (32 * WM + (GATED ? 2 : 1) * MM_COLS) * MM_PITCH * sizeof(__nv_bfloat16);
    static bool set = false;
    if (!set) {
        if (cudaFuncSetAttribute(moe_gemm_mma_kernel<TO, GATED, WM>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) !=
            cudaSuccess)
            return MU_ERR_LAUNCH;
        set = true;
    }
    return launch_pdl(moe_gemm_mma_kernel<TO, GATED, WM>, grid, dim3(MM_THREADS), smem, s, 1, x, ldx, pair_of, top, w1, w2,
                      expert_stride, ldw, tile_info, n_tiles, n, k, out, ldo, n_rows, x_group_offset, out_group_offset, gate,
                      ldg, act);
}

}  // namespace mu

// As mu_moe_gemm for bfloat16 operands whose rows start on 16-byte boundaries (k, ldx, ldw multiples of 8).
MU_EXPORT int mu_moe_gemm_mma(const void* x, long long ldx, const int* pair_of, int top, const void* w1, const void* w2,
                              long long expert_stride, long long ldw, const int* tile_info, const int* n_tiles,
                              int max_tiles, int tile_rows, int n, int k, void* out, long long ldo, int out_bf16,
                              void* stream, int act) {
    if (max_tiles <= 0) return MU_OK;
    if (!x || !w1 || !tile_info || !n_tiles || !out || n <= 0 || k <= 0 || (pair_of && top <= 0) ||
        (tile_rows != 32 && tile_rows != 64))
        return MU_ERR_BAD_ARGUMENT;
    if (k % 8 || ldx % 8 || ldw % 8 || expert_stride % 8 || ((uintptr_t)x & 15) || ((uintptr_t)w1 & 15) || ((uintptr_t)w2 & 15))
        return MU_ERR_ALIGNMENT;
    if (act != mu::ACT_NONE && act != mu::ACT_RELU2) return MU_ERR_BAD_ARGUMENT;
    cudaStream_t s = (cudaStream_t)stream;
    const dim3 grid(max_tiles, (n + mu::MM_COLS - 1) / mu::MM_COLS);
    typedef __nv_bfloat16 bf;
#define MU_MM(TO, G)                                                                                                \
    return tile_rows == 64                                                                                          \
               ? mu::launch_moe_mma<TO, G, 2>(grid, s, (const bf*)x, ldx, pair_of, top, (const bf*)w1, (const bf*)w2, \
                                              expert_stride, ldw, tile_info, n_tiles, n, k, (TO*)out, ldo, 0, 0, 0,  \
                                              nullptr, 0, act)                                                      \
               : mu::launch_moe_mma<TO, G, 1>(grid, s, (const bf*)x, ldx, pair_of, top, (const bf*)w1, (const bf*)w2, \
                                              expert_stride, ldw, tile_info, n_tiles, n, k, (TO*)out, ldo, 0, 0, 0,  \
                                              nullptr, 0, act)
    if (w2) {
        if (out_bf16) MU_MM(bf, true);
        MU_MM(float, true);
    }
    if (out_bf16) MU_MM(bf, false);
    MU_MM(float, false);
#undef MU_MM
}

// out[t, g, :] = W[g] x[t, g, :] for n_rows rows t and n_groups groups g (heads): x [n_rows][ldx] with group g's k
// inputs at column g * x_group_offset; w [n_groups][n][k] (row stride ldw, group stride w_group_stride); out
// [n_rows][ldo] with group g's n outputs at column g * out_group_offset.  bfloat16 operands, rows and slices
// starting on 16-byte boundaries; out bfloat16 or float32.  gate (bfloat16, laid out as out, row stride ldg; may be
// null): out *= sigmoid(gate).
MU_EXPORT int mu_heads_gemm(const void* x, long long ldx, long long x_group_offset, const void* w,
                            long long w_group_stride, long long ldw, int n_rows, int n_groups, int n, int k, void* out,
                            long long ldo, long long out_group_offset, int out_bf16, const void* gate, long long ldg,
                            void* stream) {
    if (n_rows <= 0 || n_groups <= 0) return MU_OK;
    if (!x || !w || !out || n <= 0 || k <= 0 || n_groups > 65535) return MU_ERR_BAD_ARGUMENT;
    if (k % 8 || ldx % 8 || ldw % 8 || w_group_stride % 8 || x_group_offset % 8 || ((uintptr_t)x & 15) || ((uintptr_t)w & 15))
        return MU_ERR_ALIGNMENT;
    cudaStream_t s = (cudaStream_t)stream;
    const int tile_rows = n_rows > 32 ? 64 : 32;
    const dim3 grid((n_rows + tile_rows - 1) / tile_rows, (n + mu::MM_COLS - 1) / mu::MM_COLS, n_groups);
    typedef __nv_bfloat16 bf;
#define MU_HG(TO, WM)                                                                                                  \
    return mu::launch_moe_mma<TO, false, WM>(grid, s, (const bf*)x, ldx, nullptr, 1, (const bf*)w, nullptr,             \
                                             w_group_stride, ldw, nullptr, nullptr, n, k, (TO*)out, ldo, n_rows,       \
                                             x_group_offset, out_group_offset, (const bf*)gate, ldg)
    if (out_bf16) {
        if (tile_rows == 64) MU_HG(bf, 2);
        MU_HG(bf, 1);
    }
    if (tile_rows == 64) MU_HG(float, 2);
    MU_HG(float, 1);
#undef MU_HG
}
