// Attention of single decoded tokens over the paged cache, split over the keys.
//
// grid = (splits, kv-head tiles, tokens).  A block handles one token, one key-value head (up to
// G_TILE of the query heads that read it; a larger group takes several blocks) and one run of
// SPLIT keys whose boundaries are multiples of SPLIT in absolute position, so that the sums of a
// (request, position) do not depend on the batch.  The group's query heads share every key and
// value load.  Each block leaves an unnormalised partial (max, sum, sum of p*v); the block that
// finishes last for its (token, kv-head tile) adds the partials in split order and writes the
// output.  There is no waiting on other blocks: the last one to arrive does the work.
//
// Scores are q.k * scale with the scale applied after the sum; softmax with the maximum taken
// out; everything in float32 (engine/src/model.c:932-956; the reference's decode kernel splits
// the keys the same way, engine/src/model_cuda.cu:942-1067).
//
// Scratch (global memory beyond inputs and outputs), sized for `tokens` and `max_splits`:
//   part_o  float [tokens][nh][max_splits][hd]      part_ml  float [tokens][nh][max_splits][2]
//   (indexed by the token's place in the launch's list, not by its index in the batch)
//   counters int [tokens][kv-head tiles], zero before the first launch; the kernel leaves them zero.
//
// Sizes: hd a multiple of 16 bytes' worth of elements (8 for bfloat16, 4 for float32) and at most
// 256; any number of heads and groups; any page size that is a multiple of that vector width is
// NOT required: rows are [page][k|v][kv head][slot][hd], so every row starts 16-byte aligned
// when hd does.
#include "common.cuh"

namespace vk {

constexpr int DEC_THREADS = 256;
constexpr int DEC_SPLIT = 256;     // keys per block: one per thread in the score phase
constexpr int DEC_G_TILE = 8;      // query heads of a group handled by one block
constexpr int DEC_MAX_HD = 256;

__device__ __forceinline__ void dec_cp_async16(void* dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}

// ASYNC: the split's keys and values are first copied into shared memory with cp.async, all of them at once
// (one trip to memory for both), and the two phases read them there; otherwise the phases read global memory.
template <typename T, bool ASYNC>
__global__ void __launch_bounds__(DEC_THREADS, 2) attention_decode_kernel(
    const T* __restrict__ q, const T* __restrict__ cache, const int32_t* __restrict__ block_tables,
    const int32_t* __restrict__ token_seg, const int32_t* __restrict__ positions, const int32_t* __restrict__ tok_list,
    T* __restrict__ out, float* __restrict__ part_o, float* __restrict__ part_ml, int* __restrict__ counters, int nh, int nkv,
    int hd, int page_size, int max_blocks, int max_splits, float scale, int window) {
    constexpr int V = Vec16<T>::N;
    extern __shared__ float smem[];
    const int g = nh / nkv;
    const int tiles_per_kv = (g + DEC_G_TILE - 1) / DEC_G_TILE;
    const int split = blockIdx.x;
    const int kvh = blockIdx.y / tiles_per_kv;
    const int h0 = kvh * g + (blockIdx.y % tiles_per_kv) * DEC_G_TILE;       // first query head of this block
    const int gt = min(DEC_G_TILE, kvh * g + g - h0);                         // query heads of this block
    const int zi = blockIdx.z;                                                // index of the token in this launch: its scratch rows
    const int t = tok_list ? tok_list[zi] : zi;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;

    const int pos = positions[t];
    const int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
    // A position beyond the grid's reach (the caller broke its promise on grid_context) loses its far keys, but the
    // count below then still names launched blocks only, so the counters return to zero and no later launch is hurt.
    const int first_split = lo / DEC_SPLIT, last_split = min(pos / DEC_SPLIT, (int)gridDim.x - 1);
    if (split < first_split || split > last_split) return;
    const int n_active = last_split - first_split + 1;
    const int k0 = split * DEC_SPLIT;
    const int nkeys = min(DEC_SPLIT, pos - k0 + 1);                           // keys k0 .. k0+nkeys-1 are not after pos

    float* qs = smem;                                  // [G_TILE][hd]
    float* ps = qs + DEC_G_TILE * hd;                  // [G_TILE][SPLIT]
    float* red = ps + DEC_G_TILE * DEC_SPLIT;          // [groups][hd], groups * hd = 8 warps * 32 lanes * V
    const int lds = hd + V;                            // a staged row and 16 bytes: 16-byte reads stay free of bank conflicts
    T* sk = reinterpret_cast<T*>(red + DEC_THREADS * V);   // [SPLIT][lds]   (ASYNC only)
    T* sv = sk + DEC_SPLIT * lds;                      // [SPLIT][lds]
    __shared__ float wred[DEC_THREADS / 32][DEC_G_TILE];
    __shared__ float stat_m[DEC_G_TILE], stat_l[DEC_G_TILE];
    __shared__ int is_last;

    const int32_t* bt = block_tables + (size_t)token_seg[t] * max_blocks;
    const size_t page_stride = (size_t)2 * nkv * page_size * hd;
    const size_t v_off = (size_t)nkv * page_size * hd;
    const int key = k0 + tid;
    const bool valid = tid < nkeys && key >= lo;
    // the page of this thread's key: from the step's metadata, which no kernel writes
    const size_t my_row = valid ? (size_t)bt[key / page_size] * page_stride + ((size_t)kvh * page_size + key % page_size) * hd : 0;

    dependency_wait();                                 // q and the cache come from the kernels before this one
    let_dependents_start();

    if (ASYNC) {
        // consecutive threads take consecutive 16-byte pieces: a warp's request covers whole lines of a page
        const int ch = hd / V;
        for (int c = tid; c < DEC_SPLIT * ch; c += DEC_THREADS) {
            const int kl = c / ch, part = c - kl * ch;
            const int kk = k0 + kl;
            if (kl < nkeys && kk >= lo) {
                const T* kr = cache + (size_t)bt[kk / page_size] * page_stride + ((size_t)kvh * page_size + kk % page_size) * hd + part * V;
                dec_cp_async16(sk + kl * lds + part * V, kr);
                dec_cp_async16(sv + kl * lds + part * V, kr + v_off);
            }
        }
    }
    if (ASYNC) asm volatile("cp.async.commit_group;" ::: "memory");
    for (int i = tid; i < gt * hd; i += DEC_THREADS) qs[i] = to_f32<T>(q[((size_t)t * nh + h0) * hd + i]);
    if (ASYNC) asm volatile("cp.async.wait_group 0;" ::: "memory");
    __syncthreads();

    // ---- scores: one key per thread -------------------------------------------------------------
    float s[DEC_G_TILE];
#pragma unroll
    for (int h = 0; h < DEC_G_TILE; h++) s[h] = 0.0f;
    if (valid) {
        const T* kr = ASYNC ? sk + tid * lds : cache + my_row;
#pragma unroll 8
        for (int c = 0; c < hd; c += V) {
            float kf[V];
            load16<T>(kr + c, kf);
#pragma unroll
            for (int h = 0; h < DEC_G_TILE; h++) {
                if (h < gt) {
#pragma unroll
                    for (int i = 0; i < V; i++) s[h] = fmaf(qs[h * hd + c + i], kf[i], s[h]);
                }
            }
        }
    }
#pragma unroll
    for (int h = 0; h < DEC_G_TILE; h++) s[h] = valid ? s[h] * scale : -INFINITY;

    // block maximum of each head
#pragma unroll
    for (int h = 0; h < DEC_G_TILE; h++) {
        const float m = warp_max(s[h]);
        if (lane == 0) wred[warp][h] = m;
    }
    __syncthreads();
    if (tid < DEC_G_TILE) {
        float m = -INFINITY;
        for (int w = 0; w < DEC_THREADS / 32; w++) m = fmaxf(m, wred[w][tid]);
        stat_m[tid] = m;
    }
    __syncthreads();
    float p[DEC_G_TILE];
#pragma unroll
    for (int h = 0; h < DEC_G_TILE; h++) {
        p[h] = (valid && h < gt) ? expf(s[h] - stat_m[h]) : 0.0f;
        if (h < gt) ps[h * DEC_SPLIT + tid] = p[h];
        const float sum = warp_sum(p[h]);
        if (lane == 0) wred[warp][h] = sum;       // safe: every thread has read stat_m's inputs before the barrier above
    }
    __syncthreads();
    if (tid < DEC_G_TILE) {
        float l = 0.0f;
        for (int w = 0; w < DEC_THREADS / 32; w++) l += wred[w][tid];
        stat_l[tid] = l;
    }

    // ---- sum of p * v: a row of v is read by hd/V lanes, 16 bytes each --------------------------
    const int lpr = hd / V;                        // lanes per row
    const int rpw = 32 / lpr;                      // rows per warp per pass (lanes beyond rpw*lpr idle)
    const int r = lane / lpr, c = (lane % lpr) * V;
    const bool lane_on = r < rpw;
    const int group = warp * rpw + r;              // which partial sum this thread adds to
    const int groups = (DEC_THREADS / 32) * rpw;
    float acc[DEC_G_TILE][V];
#pragma unroll
    for (int h = 0; h < DEC_G_TILE; h++)
#pragma unroll
        for (int i = 0; i < V; i++) acc[h][i] = 0.0f;
    if (lane_on) {
        const int row_lo = lo > k0 ? lo - k0 : 0;
        constexpr int B = ASYNC ? 2 : 8;           // rows in flight per thread: from global memory all loads are issued before any is used
        for (int base = group; base < nkeys; base += B * groups) {
            float vf[B][V];
#pragma unroll
            for (int i = 0; i < B; i++) {
                const int row = base + i * groups;
                if (row < nkeys && row >= row_lo) {
                    const int kk = k0 + row;
                    const T* vr = ASYNC ? sv + row * lds
                                        : cache + (size_t)bt[kk / page_size] * page_stride + v_off + ((size_t)kvh * page_size + kk % page_size) * hd;
                    load16<T>(vr + c, vf[i]);
                } else {
#pragma unroll
                    for (int e = 0; e < V; e++) vf[i][e] = 0.0f;
                }
            }
#pragma unroll
            for (int i = 0; i < B; i++) {
                const int row = base + i * groups;
                if (row < nkeys) {
#pragma unroll
                    for (int h = 0; h < DEC_G_TILE; h++) {
                        if (h < gt) {
                            const float pv = ps[h * DEC_SPLIT + row];
#pragma unroll
                            for (int e = 0; e < V; e++) acc[h][e] = fmaf(pv, vf[i][e], acc[h][e]);
                        }
                    }
                }
            }
        }
    }
    // The partial sums of the groups meet: inside a warp by shuffles when the lanes of a row are a power
    // of two (then lanes r = 0 hold the warp's sum), and across warps (or across all groups otherwise) in
    // shared memory, one head at a time, in a fixed order.
    const bool pow2 = (lpr & (lpr - 1)) == 0;
    if (pow2) {
#pragma unroll
        for (int h = 0; h < DEC_G_TILE; h++) {
            if (h < gt) {
#pragma unroll
                for (int e = 0; e < V; e++) {
                    float v = acc[h][e];
                    for (int o = lpr; o < 32; o <<= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
                    acc[h][e] = v;
                }
            }
        }
    }
    const int parts = pow2 ? DEC_THREADS / 32 : groups;       // partial sums per output element
    const int my_part = pow2 ? warp : group;
    const bool writer = pow2 ? (r == 0) : lane_on;
    const bool single = n_active == 1;
#pragma unroll
    for (int h = 0; h < DEC_G_TILE; h++) {
        if (h >= gt) break;                        // gt is the same for the whole block
        __syncthreads();
        if (writer) {
#pragma unroll
            for (int e = 0; e < V; e++) red[my_part * hd + c + e] = acc[h][e];
        }
        __syncthreads();
        for (int d = tid; d < hd; d += DEC_THREADS) {
            float o = 0.0f;
            for (int gi = 0; gi < parts; gi++) o += red[gi * hd + d];
            if (single) out[((size_t)t * nh + h0 + h) * hd + d] = from_f32<T>(o * (1.0f / stat_l[h]));
            else part_o[(((size_t)zi * nh + h0 + h) * max_splits + split) * hd + d] = o;
        }
    }
    if (single) return;
    if (tid < gt) {
        float* ml = part_ml + (((size_t)zi * nh + h0 + tid) * max_splits + split) * 2;
        ml[0] = stat_m[tid];
        ml[1] = stat_l[tid];
    }

    // ---- the last block of this (token, kv-head tile) combines ----------------------------------
    __threadfence();
    __syncthreads();
    int* counter = counters + (size_t)zi * (nkv * tiles_per_kv) + blockIdx.y;
    if (tid == 0) {
        const int old = atomicAdd(counter, 1);
        is_last = old == n_active - 1;
        if (is_last) *counter = 0;                 // ready for the next launch
    }
    __syncthreads();
    if (!is_last) return;
    __threadfence();
    // weights of the splits: w[h][sp] = exp(m_sp - m) / sum_sp(l_sp * exp(m_sp - m)); all loads of a stage
    // are issued together (the partials come from L2: __ldcg), then the sums run in split order
    float* wsp = ps;                               // [G_TILE][n_active], the scores are no longer needed
    for (int i = tid; i < gt * n_active; i += DEC_THREADS) {
        const int h = i / n_active, sp = first_split + i % n_active;
        const float2 ml = __ldcg(reinterpret_cast<const float2*>(part_ml + (((size_t)zi * nh + h0 + h) * max_splits + sp) * 2));
        red[i] = ml.x;                             // maxima
        wsp[h * DEC_SPLIT + (sp - first_split)] = ml.y;     // sums, for now
    }
    __syncthreads();
    if (tid < gt) {
        float m = -INFINITY;
        for (int j = 0; j < n_active; j++) m = fmaxf(m, red[tid * n_active + j]);
        float l = 0.0f;
        for (int j = 0; j < n_active; j++) {
            const float e = expf(red[tid * n_active + j] - m);
            l += wsp[tid * DEC_SPLIT + j] * e;
            wsp[tid * DEC_SPLIT + j] = e;
        }
        stat_l[tid] = 1.0f / l;
    }
    __syncthreads();
    for (int i = tid; i < gt * hd; i += DEC_THREADS) {
        const int h = i / hd, d = i % hd;
        const float* po = part_o + (((size_t)zi * nh + h0 + h) * max_splits + first_split) * hd + d;
        float o = 0.0f;
        int j = 0;
        for (; j + 4 <= n_active; j += 4) {
            const float a0 = __ldcg(po + (size_t)j * hd), a1 = __ldcg(po + (size_t)(j + 1) * hd);
            const float a2 = __ldcg(po + (size_t)(j + 2) * hd), a3 = __ldcg(po + (size_t)(j + 3) * hd);
            o += a0 * wsp[h * DEC_SPLIT + j];
            o += a1 * wsp[h * DEC_SPLIT + j + 1];
            o += a2 * wsp[h * DEC_SPLIT + j + 2];
            o += a3 * wsp[h * DEC_SPLIT + j + 3];
        }
        for (; j < n_active; j++) o += __ldcg(po + (size_t)j * hd) * wsp[h * DEC_SPLIT + j];
        out[((size_t)t * nh + h0 + h) * hd + d] = from_f32<T>(o * stat_l[h]);
    }
}

// attention_decode_mma.cu: the bfloat16 tensor-core form for head sizes 16, 32, 64, 96, 128 (same scratch, same combine).
int launch_decode_mma(const void* q, const void* cache, const int32_t* bt, const int32_t* token_seg, const int32_t* positions,
                      const int32_t* tok_list, void* out, float* part_o, float* part_ml, int* counters, int n_tokens, int nh, int nkv,
                      int hd, int page_size, int max_blocks, int splits, int grid_splits, int counter_tiles, float scale, int window,
                      cudaStream_t stream);

// attention_decode_tma.cu: the persistent kernel for large launches (bfloat16, head size 64).
bool decode_tma_takes(int n_tokens, int nh, int nkv, int hd, int page_size, int pages, int grid_splits, const void* q, const void* cache,
                      const int* error);
int launch_decode_tma(const void* q, const void* cache, const int32_t* bt, const int32_t* token_seg, const int32_t* positions,
                      const int32_t* tok_list, void* out, float* part_o, float* part_ml, int* counters, int n_tokens, int nh, int nkv,
                      int page_size, int pages, int max_blocks, int splits, int grid_splits, int counter_tiles, float scale, int window,
                      int* error, cudaStream_t stream);

}  // namespace vk

using namespace vk;

// Bytes of scratch for `tokens` decoded tokens: part_o, part_ml and counters, in that order, each 256-byte aligned.
VK_API size_t vk_attention_decode_scratch_bytes(int tokens, int nh, int nkv, int hd, int max_context) {
    const size_t splits = (size_t)(max_context + DEC_SPLIT - 1) / DEC_SPLIT;
    const size_t g = nh / nkv, tiles = nkv * ((g + DEC_G_TILE - 1) / DEC_G_TILE);
    auto up = [](size_t b) { return (b + 255) / 256 * 256; };
    return up((size_t)tokens * nh * splits * hd * 4) + up((size_t)tokens * nh * splits * 2 * 4) + up((size_t)tokens * tiles * 4);
}

// q, out [all tokens, nh*hd]; tok_list [n_tokens] names the tokens to run (null: tokens 0..n_tokens-1).
// scratch: vk_attention_decode_scratch_bytes(scratch_tokens, ..., max_context) bytes whose counters part (the
// last) was zero before the first launch.  max_context fixes the layout of the scratch; grid_context
// (<= max_context) bounds every position + 1 of this launch and sizes the grid (a captured graph keeps it).
// pages: pages of the layer's cache (0: not known; only the kernel that streams the pages through TMA needs it);
// error: a word a kernel with bounded waits sets when a wait runs out (null: such kernels are not chosen).
VK_API int vk_attention_decode(const void* q, const void* cache, const int32_t* block_tables, const int32_t* token_seg,
                               const int32_t* positions, const int32_t* tok_list, void* out, void* scratch, int scratch_tokens,
                               int n_tokens, int nh, int nkv, int hd, int page_size, int pages, int max_blocks, int max_context,
                               int grid_context, float scale, int window, int dtype, int* error, cudaStream_t stream) {
    if (n_tokens <= 0) return VK_OK;
    if (nh <= 0 || nkv <= 0 || nh % nkv != 0 || hd <= 0 || page_size <= 0 || max_blocks <= 0 || window < 0 || max_context <= 0 ||
        grid_context <= 0 || grid_context > max_context)
        return VK_BAD_SHAPE;
    const int vec = dtype == 0 ? 4 : 8;
    if (hd % vec != 0) return VK_BAD_SHAPE;
    if (hd > DEC_MAX_HD || hd / vec > 32 || n_tokens > scratch_tokens || n_tokens > 65535 || max_context > 128 * DEC_SPLIT)
        return VK_TOO_LARGE;
    if (((uintptr_t)cache % 16) || ((uintptr_t)scratch % 16) || ((uintptr_t)q % 4)) return VK_BAD_ALIGNMENT;
    const int splits = (max_context + DEC_SPLIT - 1) / DEC_SPLIT;
    const int grid_splits = (grid_context + DEC_SPLIT - 1) / DEC_SPLIT;
    const int g = nh / nkv, tiles = nkv * ((g + DEC_G_TILE - 1) / DEC_G_TILE);
    auto up = [](size_t b) { return (b + 255) / 256 * 256; };
    char* base = (char*)scratch;
    float* part_o = (float*)base;
    float* part_ml = (float*)(base + up((size_t)scratch_tokens * nh * splits * hd * 4));
    int* counters = (int*)((char*)part_ml + up((size_t)scratch_tokens * nh * splits * 2 * 4));
    if (dtype == 1 && decode_tma_takes(n_tokens, nh, nkv, hd, page_size, pages, grid_splits, q, cache, error))
        return launch_decode_tma(q, cache, block_tables, token_seg, positions, tok_list, out, part_o, part_ml, counters, n_tokens, nh, nkv,
                                 page_size, pages, max_blocks, splits, grid_splits, tiles, scale, window, error, stream);
    if (dtype == 1 && (hd == 16 || hd == 32 || hd == 64 || hd == 96 || hd == 128) && ((uintptr_t)q % 16 == 0))
        return launch_decode_mma(q, cache, block_tables, token_seg, positions, tok_list, out, part_o, part_ml, counters, n_tokens, nh,
                                 nkv, hd, page_size, max_blocks, splits, grid_splits, tiles, scale, window, stream);
    const size_t smem_base = (size_t)(DEC_G_TILE * hd + DEC_G_TILE * DEC_SPLIT + DEC_THREADS * vec) * sizeof(float);
    const size_t smem_async = smem_base + (size_t)2 * DEC_SPLIT * (hd + vec) * (dtype == 0 ? 4 : 2);
    const bool async = smem_async <= 100 * 1024;        // two blocks a multiprocessor
    const size_t smem = async ? smem_async : smem_base;
    dim3 grid(grid_splits, tiles, n_tokens);
#define GO(T, A)                                                                                                                     \
    {                                                                                                                                \
        auto kern = attention_decode_kernel<T, A>;                                                                                   \
        if (smem > 48 * 1024) {                                                                                                      \
            cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);                      \
            if (e != cudaSuccess) return (int)e;                                                                                     \
        }                                                                                                                            \
        return launch_dependent(kern, grid, dim3(DEC_THREADS), smem, stream, (const T*)q, (const T*)cache, block_tables, token_seg, \
                                positions, tok_list, (T*)out, part_o, part_ml, counters, nh, nkv, hd, page_size, max_blocks, splits, \
                                scale, window);                                                                                      \
    }
    if (dtype == 0) {
        if (async) GO(float, true) else GO(float, false)
    } else {
        if (async) GO(__nv_bfloat16, true) else GO(__nv_bfloat16, false)
    }
#undef GO
    return launch_status();
}

// ---------------------------------------------------------------------------------------------------------
// The variant that allocates nothing (see attention_decode_static.h).
// ---------------------------------------------------------------------------------------------------------
#include <mutex>

#include "attention_decode_static.h"

// The library's own scratch.  In host code this name is only a handle for cudaGetSymbolAddress: it is not a
// device pointer, and a kernel given it directly would read the wrong memory.
static __device__ __align__(256) unsigned char vk_decode_static_scratch[VK_DECODE_STATIC_SCRATCH_BYTES];

static void* decode_static_scratch_address(int* status) {
    static std::mutex lock;
    static void* address[64] = {};                 // per device
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) { *status = (int)e; return nullptr; }
    if (dev < 0 || dev >= 64) { *status = VK_TOO_LARGE; return nullptr; }
    std::lock_guard<std::mutex> guard(lock);
    if (!address[dev]) {
        void* p = nullptr;
        e = cudaGetSymbolAddress(&p, vk_decode_static_scratch);      // with device `dev` current: its copy of the array
        if (e != cudaSuccess) { *status = (int)e; return nullptr; }
        address[dev] = p;
    }
    *status = VK_OK;
    return address[dev];
}

VK_API int vk_attention_decode_static(const void* q, const void* cache, const int32_t* block_tables, const int32_t* token_seg,
                                      const int32_t* positions, const int32_t* tok_list, void* out, int n_tokens, int nh, int nkv,
                                      int hd, int page_size, int max_blocks, int max_context, float scale, int window, int dtype,
                                      cudaStream_t stream) {
    if (n_tokens <= 0) return VK_OK;
    if (nh <= 0 || nkv <= 0 || nh % nkv != 0 || hd <= 0 || page_size <= 0 || max_blocks <= 0 || window < 0 || max_context <= 0)
        return VK_BAD_SHAPE;
    const int vec = dtype == 0 ? 4 : 8;
    if (hd % vec != 0) return VK_BAD_SHAPE;
    if (hd > DEC_MAX_HD || hd / vec > 32 || n_tokens > 65535 || max_context > 128 * DEC_SPLIT) return VK_TOO_LARGE;
    if (((uintptr_t)cache % 16) || ((uintptr_t)q % 4)) return VK_BAD_ALIGNMENT;
    // the partial results of this launch must fit the array: refuse before anything runs
    if (vk_attention_decode_scratch_bytes(n_tokens, nh, nkv, hd, max_context) > VK_DECODE_STATIC_SCRATCH_BYTES) return VK_TOO_LARGE;
    int status = VK_OK;
    char* base = (char*)decode_static_scratch_address(&status);
    if (!base) return status;
    const int splits = (max_context + DEC_SPLIT - 1) / DEC_SPLIT;
    const int g = nh / nkv, tiles = nkv * ((g + DEC_G_TILE - 1) / DEC_G_TILE);
    auto up = [](size_t b) { return (b + 255) / 256 * 256; };
    float* part_o = (float*)base;
    float* part_ml = (float*)(base + up((size_t)n_tokens * nh * splits * hd * 4));
    int* counters = (int*)((char*)part_ml + up((size_t)n_tokens * nh * splits * 2 * 4));
    // the array keeps the last call's bytes, laid out for that call's sizes: the counters start at zero
    cudaError_t e = cudaMemsetAsync(counters, 0, (size_t)n_tokens * tiles * sizeof(int), stream);
    if (e != cudaSuccess) return (int)e;
    const size_t smem_base = (size_t)(DEC_G_TILE * hd + DEC_G_TILE * DEC_SPLIT + DEC_THREADS * vec) * sizeof(float);
    const size_t smem_async = smem_base + (size_t)2 * DEC_SPLIT * (hd + vec) * (dtype == 0 ? 4 : 2);
    const bool async = smem_async <= 100 * 1024;
    const size_t smem = async ? smem_async : smem_base;
    dim3 grid(splits, tiles, n_tokens);
#define GO(T, A)                                                                                                              \
    {                                                                                                                         \
        auto kern = attention_decode_kernel<T, A>;                                                                            \
        if (smem > 48 * 1024) {                                                                                               \
            e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);                           \
            if (e != cudaSuccess) return (int)e;                                                                              \
        }                                                                                                                     \
        kern<<<grid, DEC_THREADS, smem, stream>>>((const T*)q, (const T*)cache, block_tables, token_seg, positions, tok_list, \
                                                  (T*)out, part_o, part_ml, counters, nh, nkv, hd, page_size, max_blocks,     \
                                                  splits, scale, window);                                                     \
    }
    if (dtype == 0) {
        if (async) GO(float, true) else GO(float, false)
    } else {
        if (async) GO(__nv_bfloat16, true) else GO(__nv_bfloat16, false)
    }
#undef GO
    return launch_status();
}
