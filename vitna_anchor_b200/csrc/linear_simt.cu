// Matrix products on CUDA cores: out[M, N] = x[M, K] * W[N, K]^T.
//
// These are the engine's true-32-bit products and the bfloat16 path's
// products at sizes its tensor-core kernels do not take.  Inputs are widened
// exactly, every product and sum is float32 (fmaf), and the order in which an
// output element's K terms are added depends only on K and on which of the two
// kernels runs, never on M, on the position of the row in the batch, or on
// the grid: a row's result does not change with what else is in the batch.
//
// Output modes: 0 = store in the input type, 1 = store float32,
//               2 = add into a float32 output (the residual sum).
#include "common.cuh"

namespace vk {

enum { OUT_SAME = 0, OUT_F32 = 1, OUT_ACC_F32 = 2 };

template <typename T, int MODE>
__device__ __forceinline__ void store_out(void* out, size_t idx, float v) {
    if (MODE == OUT_SAME) ((T*)out)[idx] = from_f32<T>(v);
    else if (MODE == OUT_F32) ((float*)out)[idx] = v;
    else ((float*)out)[idx] += v;
}

// 64x64 output tile, K in slabs of 16, 256 threads, 4x4 outputs per thread.
// (The reference's prompt GEMM has the same tile shape, engine/src/model_cuda.cu:2579-2641.)
constexpr int TM = 64, TN = 64, TK = 16;

template <typename T, int MODE>
__global__ void __launch_bounds__(256) gemm_tile_kernel(const T* __restrict__ x, const T* __restrict__ w, void* __restrict__ out,
                                                        int M, int N, int K, int ldx) {
    __shared__ float xs[TK][TM + 4];
    __shared__ float ws[TK][TN + 4];
    const int m0 = blockIdx.y * TM, n0 = blockIdx.x * TN;
    const int tx = threadIdx.x % 16, ty = threadIdx.x / 16;
    float acc[4][4] = {};
    for (int k0 = 0; k0 < K; k0 += TK) {
        // 64 rows x 16 k of each operand: 1024 elements, 4 per thread
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const int e = threadIdx.x + i * 256;
            const int r = e / TK, kk = e % TK;
            const int gm = m0 + r, gn = n0 + r, gk = k0 + kk;
            xs[kk][r] = (gm < M && gk < K) ? to_f32<T>(x[(size_t)gm * ldx + gk]) : 0.0f;
            ws[kk][r] = (gn < N && gk < K) ? to_f32<T>(w[(size_t)gn * K + gk]) : 0.0f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < TK; kk++) {
            float a[4], b[4];
#pragma unroll
            for (int i = 0; i < 4; i++) a[i] = xs[kk][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; j++) b[j] = ws[kk][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; i++)
#pragma unroll
                for (int j = 0; j < 4; j++) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const int gm = m0 + ty * 4 + i;
        if (gm >= M) continue;
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const int gn = n0 + tx * 4 + j;
            if (gn < N) store_out<T, MODE>(out, (size_t)gm * N + gn, acc[i][j]);
        }
    }
}

// Few rows (M <= ROWS): a warp per output column streams that column's weight
// row once, 16 bytes per lane per load, and keeps one sum per input row.
// Each lane's partial sum runs over k = lane*VEC + 32*VEC*i (+0..VEC-1) in
// increasing order; the 32 partial sums meet in a fixed shuffle tree.
template <typename T, int MODE, int ROWS, bool VECTOR>
__global__ void __launch_bounds__(256) gemv_rows_kernel(const T* __restrict__ x, const T* __restrict__ w, void* __restrict__ out,
                                                        int M, int N, int K, int ldx) {
    constexpr int V = Vec16<T>::N;
    const int lane = threadIdx.x & 31;
    const int warps_per_block = blockDim.x >> 5;
    for (int n = blockIdx.x * warps_per_block + (threadIdx.x >> 5); n < N; n += gridDim.x * warps_per_block) {
        const T* wr = w + (size_t)n * K;
        float acc[ROWS];
#pragma unroll
        for (int m = 0; m < ROWS; m++) acc[m] = 0.0f;
        if (VECTOR) {
            for (int k = lane * V; k < K; k += 32 * V) {
                float wf[V];
                load16<T>(wr + k, wf);
#pragma unroll
                for (int m = 0; m < ROWS; m++) {
                    if (m < M) {
                        float xf[V];
                        load16<T>(x + (size_t)m * ldx + k, xf);
#pragma unroll
                        for (int i = 0; i < V; i++) acc[m] = fmaf(xf[i], wf[i], acc[m]);
                    }
                }
            }
        } else {
            for (int k = lane; k < K; k += 32) {
                const float wv = to_f32<T>(wr[k]);
#pragma unroll
                for (int m = 0; m < ROWS; m++)
                    if (m < M) acc[m] = fmaf(to_f32<T>(x[(size_t)m * ldx + k]), wv, acc[m]);
            }
        }
#pragma unroll
        for (int m = 0; m < ROWS; m++) {
            const float s = warp_sum(acc[m]);
            if (lane == 0 && m < M) store_out<T, MODE>(out, (size_t)m * N + n, s);
        }
    }
}

template <typename T, int MODE>
static int launch_linear(const T* x, const T* w, void* out, int M, int N, int K, int ldx, int few_rows, cudaStream_t stream) {
    if (M <= few_rows) {
        constexpr int V = Vec16<T>::N;
        const bool vec = (K % V == 0) && (ldx % V == 0) && ((uintptr_t)x % 16 == 0) && ((uintptr_t)w % 16 == 0);
        const int blocks = (N + 7) / 8 < 148 * 8 ? (N + 7) / 8 : 148 * 8;
        if (M <= 4) {
            if (vec) gemv_rows_kernel<T, MODE, 4, true><<<blocks, 256, 0, stream>>>(x, w, out, M, N, K, ldx);
            else gemv_rows_kernel<T, MODE, 4, false><<<blocks, 256, 0, stream>>>(x, w, out, M, N, K, ldx);
        } else {
            if (vec) gemv_rows_kernel<T, MODE, 8, true><<<blocks, 256, 0, stream>>>(x, w, out, M, N, K, ldx);
            else gemv_rows_kernel<T, MODE, 8, false><<<blocks, 256, 0, stream>>>(x, w, out, M, N, K, ldx);
        }
    } else {
        dim3 grid((N + TN - 1) / TN, (M + TM - 1) / TM);
        if (grid.y > 65535) return VK_TOO_LARGE;
        gemm_tile_kernel<T, MODE><<<grid, 256, 0, stream>>>(x, w, out, M, N, K, ldx);
    }
    return launch_status();
}

}  // namespace vk

using namespace vk;

// x [M, K] with row stride ldx, w [N, K], out [M, N]; dtype 0 = float32, 1 = bfloat16.
// few_rows: batches of at most this many rows (<= 8) take the column-per-warp kernel; 0 sends
// everything through the tile kernel.
VK_API int vk_linear_simt(const void* x, const void* w, void* out, int M, int N, int K, int ldx, int dtype, int mode,
                          int few_rows, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return VK_OK;
    if (K <= 0 || ldx < K || mode < 0 || mode > 2 || few_rows < 0 || few_rows > 8) return VK_BAD_SHAPE;
#define GO(T, MODE) return launch_linear<T, MODE>((const T*)x, (const T*)w, out, M, N, K, ldx, few_rows, stream)
    if (dtype == 0) {
        if (mode == 0) GO(float, OUT_SAME);
        if (mode == 1) GO(float, OUT_F32);
        GO(float, OUT_ACC_F32);
    } else {
        if (mode == 0) GO(__nv_bfloat16, OUT_SAME);
        if (mode == 1) GO(__nv_bfloat16, OUT_F32);
        GO(__nv_bfloat16, OUT_ACC_F32);
    }
#undef GO
}
