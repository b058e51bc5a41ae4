// Matrix products for a few rows (decoding): out[M, N] = x[M, K] * W[N, K]^T with M small, fused
// with what comes before and after so that a decode layer is five launches.
//
// A block stages the M input rows in shared memory once (optionally computing the RMSNorm of
// float32 rows on the way: y = (x / sqrt(mean(x^2) + eps)) * w, engine/src/kernels.c:94-111, rounded
// to the storage type exactly as the separate norm kernel rounds it), and each warp streams two
// weight rows at a time, 16 bytes per lane per load, keeping one float32 sum per (weight row, input
// row).  Which two weight rows a warp takes ("a unit") depends on the epilogue:
//
//   SAME / F32 / ACC   rows 2u, 2u+1          store in T / store float32 / add into float32 (residual sum)
//   SWIGLU             rows u, I+u            act[m, u] = silu(gate) * up       (engine/src/ops.c:283-288)
//   ROPE               rows h*hd+j, h*hd+j+hd/2 of a q or k head: the half-split pair, rotated by the
//                      token's position and written to q_out or into the token's cache slot; or two
//                      adjacent rows of v, written to the cache as they are (engine/src/ops.c:273-281,
//                      engine/src/model.c:927-930)
//
// Values that the unfused path would have stored in T between two kernels are rounded to T at the
// same points here, so both paths agree to the rounding of a float32 sum.  A lane's partial sum
// runs over k = lane*V + 32*V*i in increasing i and the 32 partial sums meet in a fixed shuffle
// tree: an output does not depend on M or on the other rows.
#include "common.cuh"

namespace vk {

enum { EPI_SAME = 0, EPI_F32 = 1, EPI_ACC = 2, EPI_SWIGLU = 3, EPI_ROPE = 4 };
constexpr int SK_ROWS = 8;          // input rows per pass
constexpr int SK_THREADS = 256;

struct SkinnyParams {
    const void* x;               // NORM: float32 [*, K] rows of stride ldx; else T [M, K] rows of stride ldx
    const int32_t* rows;         // NORM only, optional: input row of each of the M rows
    const float* norm_w;
    float eps;
    const void* w;               // T [N, K]
    void* out;                   // see the epilogues
    int M, N, K, ldx, kc;        // kc: elements of K staged at a time
    // ROPE
    const int32_t* positions;
    const float* cos_t;
    const float* sin_t;
    const int32_t* slot;
    void* cache;
    int nh, nkv, hd, page_size;
};

template <typename T> __device__ __forceinline__ float round_to(float v) { return to_f32<T>(from_f32<T>(v)); }

// Which two weight rows unit u names.
template <int EPI>
__device__ __forceinline__ void unit_rows(const SkinnyParams& p, int u, int& r0, int& r1) {
    if (EPI == EPI_SWIGLU) { r0 = u; r1 = p.N / 2 + u; }
    else if (EPI == EPI_ROPE) {
        const int half = p.hd / 2, rot_units = (p.nh + p.nkv) * half;
        if (u < rot_units) { r0 = (u / half) * p.hd + u % half; r1 = r0 + half; }
        else { r0 = (p.nh + p.nkv) * p.hd + 2 * (u - rot_units); r1 = r0 + 1; }
    } else { r0 = 2 * u; r1 = 2 * u + 1; }
}

// Stage rows m0 .. m0+mrows of x, columns kb .. kb+kn, into xs [SK_ROWS][kc].  Called by the whole block.
// Warp w copies rows w, w+8, ...: 16-byte loads, several in flight, so that staging costs about one
// trip to memory.  With NORM the row is float32, scaled by inv_rms[row] * norm_w and rounded to T.
template <typename T> __device__ __forceinline__ void store4(T* dst, float a, float b, float c, float d);
template <> __device__ __forceinline__ void store4<float>(float* dst, float a, float b, float c, float d) {
    *reinterpret_cast<float4*>(dst) = make_float4(a, b, c, d);
}
template <> __device__ __forceinline__ void store4<__nv_bfloat16>(__nv_bfloat16* dst, float a, float b, float c, float d) {
    __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(c, d);
    uint2 v;
    v.x = *reinterpret_cast<uint32_t*>(&lo);
    v.y = *reinterpret_cast<uint32_t*>(&hi);
    *reinterpret_cast<uint2*>(dst) = v;
}

template <typename T, bool NORM>
__device__ __forceinline__ void stage_rows(const SkinnyParams& p, T* xs, const float* inv_rms, int m0, int mrows, int kb, int kn,
                                           bool vec_ok) {
    constexpr int V = Vec16<T>::N;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    __syncthreads();
    for (int m = warp; m < mrows; m += (int)(blockDim.x >> 5)) {
        T* dst = xs + m * p.kc;
        if (NORM) {
            const int src = p.rows ? p.rows[m0 + m] : m0 + m;
            const float* xr = reinterpret_cast<const float*>(p.x) + (size_t)src * p.ldx + kb;
            const float* nw = p.norm_w + kb;
            const float inv = inv_rms[m];
            if (vec_ok) {
#pragma unroll 4
                for (int k = lane * 4; k < kn; k += 128) {
                    const float4 xv = *reinterpret_cast<const float4*>(xr + k);
                    const float4 wv = *reinterpret_cast<const float4*>(nw + k);
                    store4<T>(dst + k, (xv.x * inv) * wv.x, (xv.y * inv) * wv.y, (xv.z * inv) * wv.z, (xv.w * inv) * wv.w);
                }
            } else {
                for (int k = lane; k < kn; k += 32) dst[k] = from_f32<T>((xr[k] * inv) * nw[k]);
            }
        } else {
            const T* xr = reinterpret_cast<const T*>(p.x) + (size_t)(m0 + m) * p.ldx + kb;
            if (vec_ok) {
#pragma unroll 4
                for (int k = lane * V; k < kn; k += 32 * V) *reinterpret_cast<uint4*>(dst + k) = *reinterpret_cast<const uint4*>(xr + k);
            } else {
                for (int k = lane; k < kn; k += 32) dst[k] = xr[k];
            }
        }
    }
    __syncthreads();
}

template <typename T>
__device__ __forceinline__ void accumulate(const T* xs, int kc, const T* w0, const T* w1, int kn, int mrows, float* acc0, float* acc1) {
    constexpr int V = Vec16<T>::N;
    const int lane = threadIdx.x & 31;
#pragma unroll 2
    for (int k = lane * V; k < kn; k += 32 * V) {
        float wf0[V], wf1[V];
        load16<T>(w0 + k, wf0);
        load16<T>(w1 + k, wf1);
#pragma unroll
        for (int m = 0; m < SK_ROWS; m++) {
            if (m < mrows) {
                float xf[V];
                load16<T>(xs + m * kc + k, xf);
#pragma unroll
                for (int i = 0; i < V; i++) { acc0[m] = fmaf(xf[i], wf0[i], acc0[m]); acc1[m] = fmaf(xf[i], wf1[i], acc1[m]); }
            }
        }
    }
}

// The sums of unit u meet across the warp; lane m finishes row m0 + m.
template <typename T, int EPI>
__device__ __forceinline__ void finish_unit(const SkinnyParams& p, int u, int r0, int r1, bool has1, int m0, int mrows,
                                            const float* acc0, const float* acc1) {
    const int lane = threadIdx.x & 31;
    float a0 = 0.0f, a1 = 0.0f;
#pragma unroll
    for (int m = 0; m < SK_ROWS; m++) {
        const float s0 = warp_sum(acc0[m]), s1 = warp_sum(acc1[m]);
        if (lane == m) { a0 = s0; a1 = s1; }
    }
    if (lane >= mrows) return;
    const int m = m0 + lane;
    if (EPI == EPI_SAME) {
        T* o = reinterpret_cast<T*>(p.out) + (size_t)m * p.N;
        o[r0] = from_f32<T>(a0);
        if (has1) o[r1] = from_f32<T>(a1);
    } else if (EPI == EPI_F32) {
        float* o = reinterpret_cast<float*>(p.out) + (size_t)m * p.N;
        o[r0] = a0;
        if (has1) o[r1] = a1;
    } else if (EPI == EPI_ACC) {
        float* o = reinterpret_cast<float*>(p.out) + (size_t)m * p.N;
        o[r0] += a0;
        if (has1) o[r1] += a1;
    } else if (EPI == EPI_SWIGLU) {
        const float g = round_to<T>(a0), up = round_to<T>(a1);
        reinterpret_cast<T*>(p.out)[(size_t)m * (p.N / 2) + u] = from_f32<T>((g / (1.0f + expf(-g))) * up);
    } else {  // EPI_ROPE
        const int half = p.hd / 2, rot_units = (p.nh + p.nkv) * half;
        const int s = p.slot[m];
        T* cache = reinterpret_cast<T*>(p.cache);
        const size_t page = s >= 0 ? (size_t)(s / p.page_size) : 0;
        const int off = s >= 0 ? s % p.page_size : 0;
        T* kbase = cache + page * 2 * p.nkv * p.page_size * p.hd;
        if (u < rot_units) {
            const int h = u / half, j = u % half, pos = p.positions[m];
            const float c = p.cos_t[(size_t)pos * half + j], sn = p.sin_t[(size_t)pos * half + j];
            const float a = round_to<T>(a0), b = round_to<T>(a1);
            const float ra = a * c - b * sn, rb = b * c + a * sn;
            if (h < p.nh) {
                T* qo = reinterpret_cast<T*>(p.out) + (size_t)m * p.nh * p.hd + h * p.hd;
                qo[j] = from_f32<T>(ra);
                qo[j + half] = from_f32<T>(rb);
            } else if (s >= 0) {
                T* dst = kbase + ((size_t)(h - p.nh) * p.page_size + off) * p.hd;
                dst[j] = from_f32<T>(ra);
                dst[j + half] = from_f32<T>(rb);
            }
        } else if (s >= 0) {
            const int col = 2 * (u - rot_units);          // within v
            T* vbase = kbase + (size_t)p.nkv * p.page_size * p.hd;
            T* dst = vbase + ((size_t)(col / p.hd) * p.page_size + off) * p.hd + col % p.hd;
            dst[0] = from_f32<T>(a0);
            dst[1] = from_f32<T>(a1);
        }
    }
}

template <typename T, int EPI, bool NORM>
__global__ void __launch_bounds__(SK_THREADS) skinny_linear_kernel(const SkinnyParams p) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    T* xs = reinterpret_cast<T*>(smem_raw);                 // [SK_ROWS][kc]
    __shared__ float inv_rms[SK_ROWS];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int WARPS = blockDim.x >> 5;
    const T* __restrict__ W = reinterpret_cast<const T*>(p.w);
    const int K = p.K;
    const int units = (EPI == EPI_SWIGLU) ? p.N / 2 : (p.N + 1) / 2;
    // 16-byte loads of x need aligned rows (the launcher has checked the weights and K)
    const bool vec_ok = NORM ? ((reinterpret_cast<uintptr_t>(p.x) % 16 == 0) && (p.ldx % 4 == 0) && (K % 4 == 0) && (p.kc % 4 == 0) &&
                                (reinterpret_cast<uintptr_t>(p.norm_w) % 16 == 0))
                             : ((reinterpret_cast<uintptr_t>(p.x) % 16 == 0) && (p.ldx % Vec16<T>::N == 0));

    for (int m0 = 0; m0 < p.M; m0 += SK_ROWS) {
        const int mrows = min(SK_ROWS, p.M - m0);
        if (NORM) {
            __syncthreads();             // the previous pass has read inv_rms
            for (int mr = warp; mr < mrows; mr += WARPS) {          // a warp per row: the sum of squares over the whole row
                const int src = p.rows ? p.rows[m0 + mr] : m0 + mr;
                const float* xr = reinterpret_cast<const float*>(p.x) + (size_t)src * p.ldx;
                float ss = 0.0f;
                if (vec_ok) {
#pragma unroll 4
                    for (int k = lane * 4; k < K; k += 128) {
                        const float4 v = *reinterpret_cast<const float4*>(xr + k);
                        ss = fmaf(v.x, v.x, ss); ss = fmaf(v.y, v.y, ss); ss = fmaf(v.z, v.z, ss); ss = fmaf(v.w, v.w, ss);
                    }
                } else {
                    for (int k = lane; k < K; k += 32) { const float v = xr[k]; ss = fmaf(v, v, ss); }
                }
                ss = warp_sum(ss);
                if (lane == 0) inv_rms[mr] = 1.0f / sqrtf(ss / (float)K + p.eps);
            }
        }
        if (p.kc >= K) {
            // K fits: stage once, then each warp walks over units
            stage_rows<T, NORM>(p, xs, inv_rms, m0, mrows, 0, K, vec_ok);
            for (int u = blockIdx.x * WARPS + warp; u < units; u += gridDim.x * WARPS) {
                int r0, r1;
                unit_rows<EPI>(p, u, r0, r1);
                const bool has1 = r1 < p.N;
                float acc0[SK_ROWS], acc1[SK_ROWS];
#pragma unroll
                for (int m = 0; m < SK_ROWS; m++) { acc0[m] = 0.0f; acc1[m] = 0.0f; }
                accumulate<T>(xs, p.kc, W + (size_t)r0 * K, W + (size_t)(has1 ? r1 : r0) * K, K, mrows, acc0, acc1);
                finish_unit<T, EPI>(p, u, r0, r1, has1, m0, mrows, acc0, acc1);
            }
        } else {
            // K in chunks: a warp keeps one unit's sums across the chunks (the grid gives every unit a warp)
            const int u = blockIdx.x * WARPS + warp;
            const bool on = u < units;
            int r0 = 0, r1 = 0;
            if (on) unit_rows<EPI>(p, u, r0, r1);
            const bool has1 = on && r1 < p.N;
            float acc0[SK_ROWS], acc1[SK_ROWS];
#pragma unroll
            for (int m = 0; m < SK_ROWS; m++) { acc0[m] = 0.0f; acc1[m] = 0.0f; }
            for (int kb = 0; kb < K; kb += p.kc) {
                const int kn = min(p.kc, K - kb);
                stage_rows<T, NORM>(p, xs, inv_rms, m0, mrows, kb, kn, vec_ok);
                if (on) accumulate<T>(xs, p.kc, W + (size_t)r0 * K + kb, W + (size_t)(has1 ? r1 : r0) * K + kb, kn, mrows, acc0, acc1);
            }
            if (on) finish_unit<T, EPI>(p, u, r0, r1, has1, m0, mrows, acc0, acc1);
        }
    }
}

template <typename T, int EPI, bool NORM>
static int launch_skinny(SkinnyParams p, cudaStream_t stream) {
    constexpr int V = Vec16<T>::N;
    const int kc_max = 65536 / (SK_ROWS * (int)sizeof(T));           // 64 KB of shared memory for the staged rows
    p.kc = p.K <= kc_max ? p.K : kc_max;
    const int units = (EPI == EPI_SWIGLU) ? p.N / 2 : (p.N + 1) / 2;
    // few units: fewer warps a block, so that the work spreads over the SMs (a block stages x for itself)
    int warps = (units + 147) / 148;
    warps = warps < 1 ? 1 : (warps > SK_THREADS / 32 ? SK_THREADS / 32 : warps);
    int blocks = (units + warps - 1) / warps;
    if (p.kc >= p.K && blocks > 148 * 4) blocks = 148 * 4;
    const size_t smem = (size_t)SK_ROWS * p.kc * sizeof(T);
    (void)V;
    auto kern = skinny_linear_kernel<T, EPI, NORM>;
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
    }
    kern<<<blocks, 32 * warps, smem, stream>>>(p);
    return launch_status();
}

template <typename T, bool NORM>
static int dispatch_epi(int epi, const SkinnyParams& p, cudaStream_t stream) {
    switch (epi) {
        case EPI_SAME: return launch_skinny<T, EPI_SAME, NORM>(p, stream);
        case EPI_F32: return launch_skinny<T, EPI_F32, NORM>(p, stream);
        case EPI_ACC: return launch_skinny<T, EPI_ACC, NORM>(p, stream);
        case EPI_SWIGLU: return launch_skinny<T, EPI_SWIGLU, NORM>(p, stream);
        case EPI_ROPE: return launch_skinny<T, EPI_ROPE, NORM>(p, stream);
    }
    return VK_BAD_SHAPE;
}

}  // namespace vk

using namespace vk;

// x: float32 rows when norm_w is given (the RMSNorm is fused; `rows` may gather them), else rows of the
// weights' type.  w [N, K].  epi 0/1/2: out [M, N] (T / float32 / float32 +=); 3: out [M, N/2] = silu(gate)*up
// with gate rows 0..N/2-1 and up rows N/2..N-1 of w; 4: out = q_out [M, nh*hd], k and v go into `cache`
// (one layer: [pages][2][nkv][page_size][hd]) at slot[m]; needs N == (nh+2*nkv)*hd and tables [*, hd/2].
// K and ldx must be multiples of 16 bytes' worth of elements; M at most 64.
VK_API int vk_linear_skinny(const void* x, const int32_t* rows, const float* norm_w, float eps, const void* w, void* out, int M,
                            int N, int K, int ldx, int epi, const int32_t* positions, const float* cos_t, const float* sin_t,
                            const int32_t* slot, void* cache, int nh, int nkv, int hd, int page_size, int dtype,
                            cudaStream_t stream) {
    if (M <= 0 || N <= 0) return VK_OK;
    if (K <= 0 || ldx < K || epi < 0 || epi > 4) return VK_BAD_SHAPE;
    if (M > 64) return VK_TOO_LARGE;
    const int vec = dtype == 0 ? 4 : 8;
    if (K % vec != 0 || (!norm_w && ldx % vec != 0)) return VK_BAD_SHAPE;
    if (((uintptr_t)w % 16) || (!norm_w && ((uintptr_t)x % 16))) return VK_BAD_ALIGNMENT;
    if (epi == EPI_SWIGLU && (N % 2)) return VK_BAD_SHAPE;
    if (epi == EPI_ROPE) {
        if (nh <= 0 || nkv <= 0 || hd <= 0 || (hd % 2) || page_size <= 0 || N != (nh + 2 * nkv) * hd || !positions || !cos_t || !sin_t ||
            !slot || !cache)
            return VK_BAD_SHAPE;
    }
    SkinnyParams p{x, rows, norm_w, eps, w, out, M, N, K, ldx, 0, positions, cos_t, sin_t, slot, cache, nh, nkv, hd, page_size};
    if (dtype == 0) return norm_w ? dispatch_epi<float, true>(epi, p, stream) : dispatch_epi<float, false>(epi, p, stream);
    return norm_w ? dispatch_epi<__nv_bfloat16, true>(epi, p, stream) : dispatch_epi<__nv_bfloat16, false>(epi, p, stream);
}
