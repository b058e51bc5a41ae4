// Token-wise kernels: embedding rows, RMSNorm, rotation of q and k with the
// write of k and v into the paged cache, and SiLU(gate) * up.
//
// All arithmetic is float32.  T is the storage type of activations, weights
// and cache (float or __nv_bfloat16); the residual stream is always float32.
#include "common.cuh"

namespace vk {

// x[t, :] = widen(table[ids[t], :])          (engine/src/model.c:893-895)
template <typename T>
__global__ void embed_rows_kernel(const T* __restrict__ table, const int32_t* __restrict__ ids,
                                  float* __restrict__ x, int hidden, int vocab) {
    const int t = blockIdx.x;
    int id = ids[t];
    if (id < 0 || id >= vocab) id = 0;  // the host has checked the range; never read outside the table
    const T* row = table + (size_t)id * hidden;
    float* out = x + (size_t)t * hidden;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) out[i] = to_f32<T>(row[i]);
}

// y_i = (x_i * (1 / sqrt(sum(x^2)/n + eps))) * w_i    (engine/src/kernels.c:94-111)
// Four consecutive values in one store (the address is aligned to four values).
template <typename T> __device__ __forceinline__ void store4(T* p, float a, float b, float c, float d);
template <> __device__ __forceinline__ void store4<float>(float* p, float a, float b, float c, float d) {
    *reinterpret_cast<float4*>(p) = make_float4(a, b, c, d);
}
template <> __device__ __forceinline__ void store4<__nv_bfloat16>(__nv_bfloat16* p, float a, float b, float c, float d) {
    __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(c, d);
    uint2 v;
    v.x = *reinterpret_cast<uint32_t*>(&lo);
    v.y = *reinterpret_cast<uint32_t*>(&hi);
    *reinterpret_cast<uint2*>(p) = v;
}

// A warp per output row (eight rows a block): 16-byte loads when the rows allow, the 32 partial sums meet in a
// fixed shuffle tree.  `rows` (optional) names the input row of each output row.
template <typename T>
__global__ void __launch_bounds__(256) rmsnorm_rows_kernel(const float* __restrict__ x, const float* __restrict__ w,
                                                           const int32_t* __restrict__ rows, T* __restrict__ y, int out_rows, int n, float eps) {
    const int lane = threadIdx.x & 31;
    const int r = blockIdx.x * 8 + (threadIdx.x >> 5);
    dependency_wait();
    let_dependents_start();
    if (r >= out_rows) return;
    const float* in = x + (size_t)(rows ? rows[r] : r) * n;
    T* out = y + (size_t)r * n;
    const bool vec = (n % 4 == 0) && (reinterpret_cast<uintptr_t>(in) % 16 == 0) && (reinterpret_cast<uintptr_t>(w) % 16 == 0) &&
                     (reinterpret_cast<uintptr_t>(out) % (4 * sizeof(T)) == 0);
    float ss = 0.0f;
    constexpr int KEEP = 16;                       // rows of up to 128 * KEEP values stay in registers between the two passes
    if (vec && n <= 128 * KEEP) {
        float4 v[KEEP];
#pragma unroll
        for (int j = 0; j < KEEP; j++) {
            const int i = lane * 4 + j * 128;
            v[j] = i < n ? *reinterpret_cast<const float4*>(in + i) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        }
#pragma unroll
        for (int j = 0; j < KEEP; j++) {           // the same order of sums as the loop below
            if (lane * 4 + j * 128 < n) { ss = fmaf(v[j].x, v[j].x, ss); ss = fmaf(v[j].y, v[j].y, ss); ss = fmaf(v[j].z, v[j].z, ss); ss = fmaf(v[j].w, v[j].w, ss); }
        }
        ss = warp_sum(ss);
        const float inv = 1.0f / sqrtf(ss / (float)n + eps);
#pragma unroll
        for (int j = 0; j < KEEP; j++) {
            const int i = lane * 4 + j * 128;
            if (i < n) {
                const float4 g = *reinterpret_cast<const float4*>(w + i);
                store4<T>(out + i, (v[j].x * inv) * g.x, (v[j].y * inv) * g.y, (v[j].z * inv) * g.z, (v[j].w * inv) * g.w);
            }
        }
        return;
    }
    if (vec) {
#pragma unroll 4
        for (int i = lane * 4; i < n; i += 128) {
            const float4 v = *reinterpret_cast<const float4*>(in + i);
            ss = fmaf(v.x, v.x, ss); ss = fmaf(v.y, v.y, ss); ss = fmaf(v.z, v.z, ss); ss = fmaf(v.w, v.w, ss);
        }
    } else {
        for (int i = lane; i < n; i += 32) { const float v = in[i]; ss = fmaf(v, v, ss); }
    }
    ss = warp_sum(ss);
    const float inv = 1.0f / sqrtf(ss / (float)n + eps);
    if (vec) {
#pragma unroll 4
        for (int i = lane * 4; i < n; i += 128) {
            const float4 v = *reinterpret_cast<const float4*>(in + i);
            const float4 g = *reinterpret_cast<const float4*>(w + i);
            store4<T>(out + i, (v.x * inv) * g.x, (v.y * inv) * g.y, (v.z * inv) * g.z, (v.w * inv) * g.w);
        }
    } else {
        for (int i = lane; i < n; i += 32) out[i] = from_f32<T>((in[i] * inv) * w[i]);
    }
}

// Half-split rotation of every q head and k head of a token, and the write of
// the rotated k and the raw v into the token's cache slot
// (engine/src/ops.c:273-281, engine/src/model.c:927-930).
//
// qkv      [tokens, (nh + 2*nkv) * hd]: q heads, then k heads, then v heads
// q_out    [tokens, nh * hd]
// cos,sin  [max_pos, rot/2] float32 host-built tables (null: no rotation)
// slot     [tokens]: page * page_size + offset of the token in this layer's cache, or -1 (no write)
// cache    one layer: [pages][2][nkv][page_size][hd]
template <typename T>
__global__ void rope_store_kernel(const T* __restrict__ qkv, const int32_t* __restrict__ positions,
                                  const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                                  const int32_t* __restrict__ slot, T* __restrict__ q_out, T* __restrict__ cache,
                                  int nh, int nkv, int hd, int rot, int page_size) {
    const int t = blockIdx.x;
    const int half = rot / 2;
    const int pos = positions[t];
    const T* in = qkv + (size_t)t * (nh + 2 * nkv) * hd;
    const int s = slot ? slot[t] : -1;
    const size_t page = s >= 0 ? (size_t)(s / page_size) : 0;
    const int off = s >= 0 ? s % page_size : 0;
    T* kbase = cache ? cache + page * 2 * nkv * page_size * hd : nullptr;
    T* vbase = cache ? kbase + (size_t)nkv * page_size * hd : nullptr;

    // rotated pairs of q and k
    const int pair_units = (nh + nkv) * half;
    for (int u = threadIdx.x; u < pair_units; u += blockDim.x) {
        const int h = u / half, j = u % half;
        const float c = cos_t[(size_t)pos * half + j], sn = sin_t[(size_t)pos * half + j];
        const float a = to_f32<T>(in[h * hd + j]), b = to_f32<T>(in[h * hd + j + half]);
        const float ra = a * c - b * sn, rb = b * c + a * sn;
        if (h < nh) {
            q_out[(size_t)t * nh * hd + h * hd + j] = from_f32<T>(ra);
            q_out[(size_t)t * nh * hd + h * hd + j + half] = from_f32<T>(rb);
        } else if (s >= 0) {
            T* dst = kbase + ((size_t)(h - nh) * page_size + off) * hd;
            dst[j] = from_f32<T>(ra);
            dst[j + half] = from_f32<T>(rb);
        }
    }
    // dimensions beyond the rotated part pass through
    const int rest = hd - rot;
    if (rest > 0) {
        for (int u = threadIdx.x; u < (nh + nkv) * rest; u += blockDim.x) {
            const int h = u / rest, d = rot + u % rest;
            const T v = in[h * hd + d];
            if (h < nh) q_out[(size_t)t * nh * hd + h * hd + d] = v;
            else if (s >= 0) kbase[((size_t)(h - nh) * page_size + off) * hd + d] = v;
        }
    }
    // v is stored as it is
    if (s >= 0) {
        const T* vin = in + (size_t)(nh + nkv) * hd;
        for (int u = threadIdx.x; u < nkv * hd; u += blockDim.x) {
            const int h = u / hd, d = u % hd;
            vbase[((size_t)h * page_size + off) * hd + d] = vin[u];
        }
    }
}

// act_i = (g_i / (1 + exp(-g_i))) * u_i       (engine/src/ops.c:283-288)
// gu [tokens, 2*inter]: gate columns, then up columns.
template <typename T>
__global__ void silu_mul_kernel(const T* __restrict__ gu, T* __restrict__ act, size_t tokens, int inter) {
    const size_t n = tokens * (size_t)inter;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        const size_t t = i / inter;
        const int c = (int)(i % inter);
        const float g = to_f32<T>(gu[t * 2 * inter + c]);
        const float u = to_f32<T>(gu[t * 2 * inter + inter + c]);
        act[i] = from_f32<T>((g / (1.0f + expf(-g))) * u);
    }
}

// y += x (float32), for parts that cannot add into the residual themselves.
__global__ void add_inplace_kernel(float* __restrict__ y, const float* __restrict__ x, size_t n) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) y[i] += x[i];
}

template <typename T>
__global__ void add_cast_inplace_kernel(float* __restrict__ y, const T* __restrict__ x, size_t n) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) y[i] += to_f32<T>(x[i]);
}

// tokens[i] = ids[src[i]] where src[i] >= 0: the ids a step's sampling left on the device become the next step's
// input tokens without a trip through the host.
__global__ void take_tokens_kernel(int32_t* __restrict__ tokens, const int32_t* __restrict__ ids, const int32_t* __restrict__ src, int n) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n && src[i] >= 0) tokens[i] = ids[src[i]];
}

}  // namespace vk

using namespace vk;

VK_API int vk_take_tokens(int32_t* tokens, const int32_t* ids, const int32_t* src, int n, cudaStream_t stream) {
    if (n <= 0) return VK_OK;
    take_tokens_kernel<<<(n + 127) / 128, 128, 0, stream>>>(tokens, ids, src, n);
    return launch_status();
}

static inline int grid_for(size_t n, int threads) {
    size_t g = (n + threads - 1) / threads;
    return (int)(g < 1 ? 1 : (g > 148 * 16 ? 148 * 16 : g));
}

// dtype: 0 = float32, 1 = bfloat16
VK_API int vk_embed_rows(const void* table, const int32_t* ids, float* x, int tokens, int hidden, int vocab, int dtype,
                         cudaStream_t stream) {
    if (tokens <= 0) return VK_OK;
    if (hidden <= 0 || vocab <= 0) return VK_BAD_SHAPE;
    if (dtype == 0) embed_rows_kernel<float><<<tokens, 128, 0, stream>>>((const float*)table, ids, x, hidden, vocab);
    else embed_rows_kernel<__nv_bfloat16><<<tokens, 128, 0, stream>>>((const __nv_bfloat16*)table, ids, x, hidden, vocab);
    return launch_status();
}

VK_API int vk_rmsnorm_rows(const float* x, const float* w, const int32_t* rows, void* y, int out_rows, int n, float eps,
                           int dtype, cudaStream_t stream) {
    if (out_rows <= 0) return VK_OK;
    if (n <= 0) return VK_BAD_SHAPE;
    const dim3 grid((out_rows + 7) / 8);
    if (dtype == 0) return launch_dependent(rmsnorm_rows_kernel<float>, grid, dim3(256), 0, stream, x, w, rows, (float*)y, out_rows, n, eps);
    return launch_dependent(rmsnorm_rows_kernel<__nv_bfloat16>, grid, dim3(256), 0, stream, x, w, rows, (__nv_bfloat16*)y, out_rows, n, eps);
}

VK_API int vk_rope_store(const void* qkv, const int32_t* positions, const float* cos_t, const float* sin_t,
                         const int32_t* slot, void* q_out, void* cache, int tokens, int nh, int nkv, int hd, int rot,
                         int page_size, int dtype, cudaStream_t stream) {
    if (tokens <= 0) return VK_OK;
    if (nh <= 0 || nkv <= 0 || hd <= 0 || rot < 0 || rot > hd || (rot & 1) || page_size <= 0) return VK_BAD_SHAPE;
    if (rot > 0 && (!cos_t || !sin_t)) return VK_BAD_SHAPE;
    if (dtype == 0)
        rope_store_kernel<float><<<tokens, 256, 0, stream>>>((const float*)qkv, positions, cos_t, sin_t, slot, (float*)q_out,
                                                              (float*)cache, nh, nkv, hd, rot, page_size);
    else
        rope_store_kernel<__nv_bfloat16><<<tokens, 256, 0, stream>>>((const __nv_bfloat16*)qkv, positions, cos_t, sin_t, slot,
                                                                      (__nv_bfloat16*)q_out, (__nv_bfloat16*)cache, nh, nkv, hd,
                                                                      rot, page_size);
    return launch_status();
}

VK_API int vk_silu_mul(const void* gu, void* act, int tokens, int inter, int dtype, cudaStream_t stream) {
    if (tokens <= 0) return VK_OK;
    if (inter <= 0) return VK_BAD_SHAPE;
    const size_t n = (size_t)tokens * inter;
    if (dtype == 0) silu_mul_kernel<float><<<grid_for(n, 256), 256, 0, stream>>>((const float*)gu, (float*)act, tokens, inter);
    else silu_mul_kernel<__nv_bfloat16><<<grid_for(n, 256), 256, 0, stream>>>((const __nv_bfloat16*)gu, (__nv_bfloat16*)act, tokens, inter);
    return launch_status();
}

// y (float32) += x, x float32 (dtype 0) or bfloat16 (dtype 1)
VK_API int vk_add_inplace(float* y, const void* x, size_t n, int dtype, cudaStream_t stream) {
    if (n == 0) return VK_OK;
    if (dtype == 0) add_inplace_kernel<<<grid_for(n, 256), 256, 0, stream>>>(y, (const float*)x, n);
    else add_cast_inplace_kernel<__nv_bfloat16><<<grid_for(n, 256), 256, 0, stream>>>(y, (const __nv_bfloat16*)x, n);
    return launch_status();
}
