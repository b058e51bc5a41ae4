// Causal attention over the paged cache, one block per (token, query head).
//
// This is the engine's attention for every size and both storage types: any
// head size, any number of heads and groups, any page size, an optional
// window.  The 32-bit path always runs it; the bfloat16 path runs it where
// the specialised kernels do not take the sizes.  A token of a prompt portion
// and a single decoded token take the same code: a query at position p of a
// request reads keys lo..p of that request through its block table
// (lo = 0, or p - window + 1 with a window).
//
// Scores are q.k * scale with the scale applied after the sum, the softmax
// takes the maximum out, sums and products are float32
// (engine/src/model.c:932-956).  Keys are taken in runs of 128 whose
// boundaries are multiples of 128 in absolute position, so the order of the
// sums of a (request, position) does not depend on how the tokens were cut
// into steps or on what else is in the batch.
#include "common.cuh"

namespace vk {

constexpr int ATT_THREADS = 128;
constexpr int ATT_MAX_ACC = 4;  // head sizes up to 4 * 128

template <typename T>
__global__ void __launch_bounds__(ATT_THREADS) attention_rows_kernel(
    const T* __restrict__ q, const T* __restrict__ cache, const int32_t* __restrict__ block_tables,
    const int32_t* __restrict__ token_seg, const int32_t* __restrict__ positions, const int32_t* __restrict__ tok_list,
    T* __restrict__ out, int nh, int nkv, int hd, int page_size, int max_blocks, float scale, int window) {
    extern __shared__ float smem[];
    float* qs = smem;                         // [hd]
    float* pr = qs + hd;                      // [128]
    float* scratch = pr + ATT_THREADS;        // [32]
    __shared__ size_t row_off[ATT_THREADS];   // element offset of each key's K row in the layer's cache

    const int t = tok_list ? tok_list[blockIdx.x] : blockIdx.x, h = blockIdx.y, tid = threadIdx.x;
    const int kvh = h / (nh / nkv);
    const int pos = positions[t];
    const int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
    const int32_t* bt = block_tables + (size_t)token_seg[t] * max_blocks;
    const size_t page_stride = (size_t)2 * nkv * page_size * hd;
    const size_t v_off = (size_t)nkv * page_size * hd;

    const T* qrow = q + ((size_t)t * nh + h) * hd;
    for (int d = tid; d < hd; d += ATT_THREADS) qs[d] = to_f32<T>(qrow[d]);
    __syncthreads();

    float m = -INFINITY, l = 0.0f;
    float acc[ATT_MAX_ACC] = {0.0f, 0.0f, 0.0f, 0.0f};

    for (int c0 = (lo / ATT_THREADS) * ATT_THREADS; c0 <= pos; c0 += ATT_THREADS) {
        const int key = c0 + tid;
        const bool valid = key >= lo && key <= pos;
        float s = -INFINITY;
        if (valid) {
            const int page = bt[key / page_size];
            const size_t off = (size_t)page * page_stride + ((size_t)kvh * page_size + key % page_size) * hd;
            row_off[tid] = off;
            const T* kr = cache + off;
            float dot = 0.0f;
            for (int d = 0; d < hd; d++) dot = fmaf(qs[d], to_f32<T>(kr[d]), dot);
            s = dot * scale;
        }
        const float cmax = block_max(s, scratch);
        const float m_new = fmaxf(m, cmax);
        const float p = valid ? expf(s - m_new) : 0.0f;
        pr[tid] = p;
        const float csum = block_sum(p, scratch);  // the barriers inside also publish pr and row_off
        const float corr = expf(m - m_new);        // 0 on the first run, where m is -inf
        l = l * corr + csum;
        m = m_new;
        const int j0 = (lo > c0 ? lo : c0) - c0;
        const int j1 = (pos < c0 + ATT_THREADS - 1 ? pos : c0 + ATT_THREADS - 1) - c0;
#pragma unroll
        for (int a = 0; a < ATT_MAX_ACC; a++) {
            const int d = tid + a * ATT_THREADS;
            if (d < hd) {
                float v = acc[a] * corr;
                for (int j = j0; j <= j1; j++) v = fmaf(pr[j], to_f32<T>(cache[row_off[j] + v_off + d]), v);
                acc[a] = v;
            }
        }
        __syncthreads();  // pr and row_off are rewritten by the next run
    }
    const float inv = 1.0f / l;
    T* orow = out + ((size_t)t * nh + h) * hd;
#pragma unroll
    for (int a = 0; a < ATT_MAX_ACC; a++) {
        const int d = tid + a * ATT_THREADS;
        if (d < hd) orow[d] = from_f32<T>(acc[a] * inv);
    }
}

}  // namespace vk

using namespace vk;

// q, out [tokens, nh*hd]; cache: one layer [pages][2][nkv][page_size][hd];
// block_tables [segments, max_blocks]; token_seg, positions [all tokens]; tok_list [tokens] names the
// tokens to run (null: 0..tokens-1).
VK_API int vk_attention_rows(const void* q, const void* cache, const int32_t* block_tables, const int32_t* token_seg,
                             const int32_t* positions, const int32_t* tok_list, void* out, int tokens, int nh, int nkv, int hd, int page_size,
                             int max_blocks, float scale, int window, int dtype, cudaStream_t stream) {
    if (tokens <= 0) return VK_OK;
    if (nh <= 0 || nkv <= 0 || nh % nkv != 0 || hd <= 0 || page_size <= 0 || max_blocks <= 0 || window < 0) return VK_BAD_SHAPE;
    if (hd > ATT_THREADS * ATT_MAX_ACC || nh > 65535) return VK_TOO_LARGE;
    const size_t smem = (size_t)(hd + ATT_THREADS + 32) * sizeof(float);
    dim3 grid(tokens, nh);
    if (dtype == 0)
        attention_rows_kernel<float><<<grid, ATT_THREADS, smem, stream>>>((const float*)q, (const float*)cache, block_tables,
                                                                          token_seg, positions, tok_list, (float*)out, nh, nkv, hd,
                                                                          page_size, max_blocks, scale, window);
    else
        attention_rows_kernel<__nv_bfloat16><<<grid, ATT_THREADS, smem, stream>>>(
            (const __nv_bfloat16*)q, (const __nv_bfloat16*)cache, block_tables, token_seg, positions, tok_list, (__nv_bfloat16*)out, nh,
            nkv, hd, page_size, max_blocks, scale, window);
    return launch_status();
}
