// Split-key decode attention in bfloat16 with the scores and p*v on the tensor cores.
//
// Same decomposition and scratch as attention_decode.cu: grid = (splits of 256 keys at absolute positions,
// kv-head tiles, tokens); each block leaves an unnormalised partial and the last block of a
// (token, kv-head tile) combines them in split order.  What differs is the arithmetic of a block: the
// query heads that share a key-value head (up to 16 a block) are the 16 rows of an m16n8k16 product.
//
//   copy      keys and values of the split into shared memory with cp.async (one trip for both)
//   scores    warp w: S[16 heads x 32 keys] = Q K^T for keys 32w .. 32w+31
//   softmax   row maximum and row sum over the split's 256 keys (through shared memory), float32
//   p * v     the probabilities go to shared memory as a high and a low bfloat16 part (p = hi + lo to
//             about 2^-17, see attention_prefill.cu); warp w computes every head's output for its own
//             slice of the head dimensions over ALL keys, so no sum across warps is needed
//
// Instantiated for head sizes 16, 32, 64, 96 and 128; attention_decode.cu takes the others and float32.
#include "common.cuh"

namespace vk {

constexpr int DM_THREADS = 256, DM_SPLIT = 256, DM_ROWS = 16;

__device__ __forceinline__ void dm_cp_async16(void* dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void dm_ldsm_x4(uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3, const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"((uint32_t)__cvta_generic_to_shared(p)));
}
__device__ __forceinline__ void dm_ldsm_x2_trans(uint32_t& r0, uint32_t& r1, const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x2.trans.shared.b16 {%0,%1}, [%2];"
                 : "=r"(r0), "=r"(r1) : "r"((uint32_t)__cvta_generic_to_shared(p)));
}
__device__ __forceinline__ void dm_mma(float* d, const uint32_t* a, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

template <int HD>
__global__ void __launch_bounds__(DM_THREADS, 2) attention_decode_mma_kernel(
    const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ cache, const int32_t* __restrict__ block_tables,
    const int32_t* __restrict__ token_seg, const int32_t* __restrict__ positions, const int32_t* __restrict__ tok_list,
    __nv_bfloat16* __restrict__ out, float* __restrict__ part_o, float* __restrict__ part_ml, int* __restrict__ counters, int nh,
    int nkv, int page_size, int max_blocks, int max_splits, int counter_tiles, float scale, int window) {
    typedef __nv_bfloat16 T;
    constexpr int LD = HD + 8;                  // padded rows: ldmatrix and 16-byte copies stay free of bank conflicts
    constexpr int LP = DM_SPLIT + 8;            // padded rows of P
    constexpr int KSTEPS = HD / 16, DBLK = HD / 8;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    T* sk = reinterpret_cast<T*>(smem_raw);     // [256][LD]
    T* sv = sk + DM_SPLIT * LD;                 // [256][LD]
    T* sq = sv + DM_SPLIT * LD;                 // [16][LD]
    T* sph = sq + DM_ROWS * LD;                 // [16][LP] high parts of p
    T* spl = sph + DM_ROWS * LP;                // [16][LP] low parts
    float* wstat = reinterpret_cast<float*>(spl + DM_ROWS * LP);   // [8 warps][16 rows]: maxima, then sums
    float* wts = wstat + 8 * DM_ROWS;           // [16][max 128 splits] weights of the combine
    __shared__ float row_m[DM_ROWS], row_l[DM_ROWS];
    __shared__ int is_last;

    const int g = nh / nkv;
    const int tiles_per_kv = (g + DM_ROWS - 1) / DM_ROWS;
    const int split = blockIdx.x;
    const int kvh = blockIdx.y / tiles_per_kv;
    const int h0 = kvh * g + (blockIdx.y % tiles_per_kv) * DM_ROWS;
    const int gt = min(DM_ROWS, kvh * g + g - h0);
    const int zi = blockIdx.z;
    const int t = tok_list ? tok_list[zi] : zi;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int gq = lane >> 2, qd = lane & 3;

    const int pos = positions[t];
    const int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
    const int first_split = lo / DM_SPLIT, last_split = pos / DM_SPLIT;
    if (split < first_split || split > last_split) return;
    const int n_active = last_split - first_split + 1;
    const int k0 = split * DM_SPLIT;
    const int nkeys = min(DM_SPLIT, pos - k0 + 1);

    const int32_t* bt = block_tables + (size_t)token_seg[t] * max_blocks;
    const size_t page_stride = (size_t)2 * nkv * page_size * HD;
    const size_t v_off = (size_t)nkv * page_size * HD;
    const int key = k0 + tid;
    const bool valid = tid < nkeys && key >= lo;
    const size_t my_row = valid ? (size_t)bt[key / page_size] * page_stride + ((size_t)kvh * page_size + key % page_size) * HD : 0;

    dependency_wait();                          // q and the cache come from the kernels before this one
    let_dependents_start();

    // ---- copy: thread = key -------------------------------------------------------------------------------
    {
        T* dk = sk + tid * LD;
        T* dv = sv + tid * LD;
        if (valid) {
            const T* kr = cache + my_row;
#pragma unroll
            for (int c = 0; c < HD; c += 8) {
                dm_cp_async16(dk + c, kr + c);
                dm_cp_async16(dv + c, kr + v_off + c);
            }
        } else {                                // never counted (p = 0), but 0 * garbage must not be NaN
#pragma unroll
            for (int c = 0; c < HD; c += 8) {
                *reinterpret_cast<uint4*>(dk + c) = make_uint4(0, 0, 0, 0);
                *reinterpret_cast<uint4*>(dv + c) = make_uint4(0, 0, 0, 0);
            }
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
        // q of this block's heads, rows beyond them zero
        for (int i = tid; i < DM_ROWS * (HD / 8); i += DM_THREADS) {
            const int r = i / (HD / 8), c = (i % (HD / 8)) * 8;
            uint4 v = make_uint4(0, 0, 0, 0);
            if (r < gt) v = *reinterpret_cast<const uint4*>(q + ((size_t)t * nh + h0 + r) * HD + c);
            *reinterpret_cast<uint4*>(sq + r * LD + c) = v;
        }
        asm volatile("cp.async.wait_group 0;" ::: "memory");
    }
    __syncthreads();

    // ---- scores of keys 32*warp .. +31: four blocks of 8 keys ---------------------------------------------
    float s[4][4];
#pragma unroll
    for (int nb = 0; nb < 4; nb++) { s[nb][0] = s[nb][1] = s[nb][2] = s[nb][3] = 0.0f; }
#pragma unroll
    for (int ks = 0; ks < KSTEPS; ks++) {
        uint32_t a[4];
        dm_ldsm_x4(a[0], a[1], a[2], a[3], sq + (lane & 15) * LD + ks * 16 + (lane >> 4) * 8);
#pragma unroll
        for (int nb2 = 0; nb2 < 2; nb2++) {
            uint32_t b0, b1, b2, b3;
            dm_ldsm_x4(b0, b1, b2, b3, sk + (warp * 32 + nb2 * 16 + (lane & 7) + ((lane >> 4) << 3)) * LD + ks * 16 + ((lane >> 3) & 1) * 8);
            dm_mma(s[nb2 * 2], a, b0, b1);
            dm_mma(s[nb2 * 2 + 1], a, b2, b3);
        }
    }
    // scale, mask; rows gq and gq+8 (heads), keys warp*32 + nb*8 + 2*qd + {0,1}
    float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int nb = 0; nb < 4; nb++) {
#pragma unroll
        for (int e = 0; e < 4; e++) {
            const int kk = k0 + warp * 32 + nb * 8 + qd * 2 + (e & 1);
            const float v = (kk <= pos && kk >= lo) ? s[nb][e] * scale : -INFINITY;
            s[nb][e] = v;
            mx[e >> 1] = fmaxf(mx[e >> 1], v);
        }
    }
#pragma unroll
    for (int r = 0; r < 2; r++) {
        mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
        mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
    }
    if (qd == 0) { wstat[warp * DM_ROWS + gq] = mx[0]; wstat[warp * DM_ROWS + gq + 8] = mx[1]; }
    __syncthreads();
    float m[2];
#pragma unroll
    for (int r = 0; r < 2; r++) {
        float v = -INFINITY;
#pragma unroll
        for (int w = 0; w < 8; w++) v = fmaxf(v, wstat[w * DM_ROWS + gq + 8 * r]);
        m[r] = v;                               // finite: the split has at least one key that every row sees
    }
    __syncthreads();                            // wstat is reused for the sums
    float rs[2] = {0.0f, 0.0f};
#pragma unroll
    for (int nb = 0; nb < 4; nb++) {
        const float p0 = expf(s[nb][0] - m[0]), p1 = expf(s[nb][1] - m[0]);
        const float p2 = expf(s[nb][2] - m[1]), p3 = expf(s[nb][3] - m[1]);
        rs[0] += p0 + p1;
        rs[1] += p2 + p3;
        const int col = warp * 32 + nb * 8 + qd * 2;
        __nv_bfloat162 h01 = __floats2bfloat162_rn(p0, p1), h23 = __floats2bfloat162_rn(p2, p3);
        *reinterpret_cast<__nv_bfloat162*>(sph + gq * LP + col) = h01;
        *reinterpret_cast<__nv_bfloat162*>(sph + (gq + 8) * LP + col) = h23;
        *reinterpret_cast<__nv_bfloat162*>(spl + gq * LP + col) =
            __floats2bfloat162_rn(p0 - __bfloat162float(h01.x), p1 - __bfloat162float(h01.y));
        *reinterpret_cast<__nv_bfloat162*>(spl + (gq + 8) * LP + col) =
            __floats2bfloat162_rn(p2 - __bfloat162float(h23.x), p3 - __bfloat162float(h23.y));
    }
#pragma unroll
    for (int r = 0; r < 2; r++) {
        rs[r] += __shfl_xor_sync(0xffffffffu, rs[r], 1);
        rs[r] += __shfl_xor_sync(0xffffffffu, rs[r], 2);
    }
    if (qd == 0) { wstat[warp * DM_ROWS + gq] = rs[0]; wstat[warp * DM_ROWS + gq + 8] = rs[1]; }
    __syncthreads();
    if (tid < DM_ROWS) {
        float l = 0.0f;
#pragma unroll
        for (int w = 0; w < 8; w++) l += wstat[w * DM_ROWS + tid];
        row_l[tid] = l;
    }
    if (warp == 0 && qd == 0) { row_m[gq] = m[0]; row_m[gq + 8] = m[1]; }

    // ---- p * v: warp w computes the 8-wide blocks of head dimensions w, w+8, ... over all 256 keys ------------------
    const bool single = n_active == 1;
    __syncthreads();                            // row_l, row_m and P are written
    for (int db = warp; db < DBLK; db += 8) {
        float o[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll 4
        for (int kk = 0; kk < DM_SPLIT / 16; kk++) {
            uint32_t ah[4], al[4], b0, b1;
            dm_ldsm_x4(ah[0], ah[1], ah[2], ah[3], sph + (lane & 15) * LP + kk * 16 + (lane >> 4) * 8);
            dm_ldsm_x4(al[0], al[1], al[2], al[3], spl + (lane & 15) * LP + kk * 16 + (lane >> 4) * 8);
            dm_ldsm_x2_trans(b0, b1, sv + (kk * 16 + (lane & 15)) * LD + db * 8);
            dm_mma(o, ah, b0, b1);
            dm_mma(o, al, b0, b1);
        }
        // rows gq, gq+8 (heads), dimensions db*8 + 2*qd + {0,1}
#pragma unroll
        for (int r = 0; r < 2; r++) {
            const int row = gq + 8 * r;
            if (row >= gt) continue;
            const int d = db * 8 + qd * 2;
            if (single) {
                const float inv = 1.0f / row_l[row];
                *reinterpret_cast<__nv_bfloat162*>(out + ((size_t)t * nh + h0 + row) * HD + d) =
                    __floats2bfloat162_rn(o[2 * r] * inv, o[2 * r + 1] * inv);
            } else {
                *reinterpret_cast<float2*>(part_o + (((size_t)zi * nh + h0 + row) * max_splits + split) * HD + d) =
                    make_float2(o[2 * r], o[2 * r + 1]);
            }
        }
    }
    if (single) return;
    if (tid < gt) {
        float* ml = part_ml + (((size_t)zi * nh + h0 + tid) * max_splits + split) * 2;
        ml[0] = row_m[tid];
        ml[1] = row_l[tid];
    }

    // ---- the last block of this (token, kv-head tile) combines ----------------------------------------------
    __threadfence();
    __syncthreads();
    int* counter = counters + (size_t)zi * counter_tiles + blockIdx.y;
    if (tid == 0) {
        const int old = atomicAdd(counter, 1);
        is_last = old == n_active - 1;
        if (is_last) *counter = 0;              // ready for the next launch
    }
    __syncthreads();
    if (!is_last) return;
    __threadfence();
    float* mxs = reinterpret_cast<float*>(sk);  // [16][n_active] maxima of the splits (the keys are no longer needed)
    for (int i = tid; i < gt * n_active; i += DM_THREADS) {
        const int h = i / n_active, sp = first_split + i % n_active;
        const float2 ml = __ldcg(reinterpret_cast<const float2*>(part_ml + (((size_t)zi * nh + h0 + h) * max_splits + sp) * 2));
        mxs[i] = ml.x;
        wts[h * 128 + (sp - first_split)] = ml.y;
    }
    __syncthreads();
    if (tid < gt) {
        float mm = -INFINITY;
        for (int j = 0; j < n_active; j++) mm = fmaxf(mm, mxs[tid * n_active + j]);
        float l = 0.0f;
        for (int j = 0; j < n_active; j++) {
            const float e = expf(mxs[tid * n_active + j] - mm);
            l += wts[tid * 128 + j] * e;
            wts[tid * 128 + j] = e;
        }
        row_l[tid] = 1.0f / l;
    }
    __syncthreads();
    for (int i = tid; i < gt * HD; i += DM_THREADS) {
        const int h = i / HD, d = i % HD;
        const float* po = part_o + (((size_t)zi * nh + h0 + h) * max_splits + first_split) * HD + d;
        float o = 0.0f;
        int j = 0;
        for (; j + 4 <= n_active; j += 4) {
            const float a0 = __ldcg(po + (size_t)j * HD), a1 = __ldcg(po + (size_t)(j + 1) * HD);
            const float a2 = __ldcg(po + (size_t)(j + 2) * HD), a3 = __ldcg(po + (size_t)(j + 3) * HD);
            o += a0 * wts[h * 128 + j];
            o += a1 * wts[h * 128 + j + 1];
            o += a2 * wts[h * 128 + j + 2];
            o += a3 * wts[h * 128 + j + 3];
        }
        for (; j < n_active; j++) o += __ldcg(po + (size_t)j * HD) * wts[h * 128 + j];
        out[((size_t)t * nh + h0 + h) * HD + d] = __float2bfloat16_rn(o * row_l[h]);
    }
}

template <int HD>
static int launch_dm(const void* q, const void* cache, const int32_t* bt, const int32_t* token_seg, const int32_t* positions,
                     const int32_t* tok_list, void* out, float* part_o, float* part_ml, int* counters, int n_tokens, int nh, int nkv,
                     int page_size, int max_blocks, int splits, int grid_splits, int counter_tiles, float scale, int window,
                     cudaStream_t stream) {
    constexpr int LD = HD + 8, LP = DM_SPLIT + 8;
    const size_t smem = (size_t)(2 * DM_SPLIT * LD + DM_ROWS * LD + 2 * DM_ROWS * LP) * 2 + (size_t)(8 * DM_ROWS + DM_ROWS * 128) * 4;
    auto kern = attention_decode_mma_kernel<HD>;
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
    }
    const int g = nh / nkv, tiles = nkv * ((g + DM_ROWS - 1) / DM_ROWS);
    return launch_dependent(kern, dim3(grid_splits, tiles, n_tokens), dim3(DM_THREADS), smem, stream, (const __nv_bfloat16*)q,
                            (const __nv_bfloat16*)cache, bt, token_seg, positions, tok_list, (__nv_bfloat16*)out, part_o, part_ml,
                            counters, nh, nkv, page_size, max_blocks, splits, counter_tiles, scale, window);
}

// Called by vk_attention_decode for bfloat16 and the head sizes built here.  Returns VK_BAD_SHAPE for other head sizes.
int launch_decode_mma(const void* q, const void* cache, const int32_t* bt, const int32_t* token_seg, const int32_t* positions,
                      const int32_t* tok_list, void* out, float* part_o, float* part_ml, int* counters, int n_tokens, int nh, int nkv,
                      int hd, int page_size, int max_blocks, int splits, int grid_splits, int counter_tiles, float scale, int window,
                      cudaStream_t stream) {
#define GO(HD)                                                                                                                   \
    return launch_dm<HD>(q, cache, bt, token_seg, positions, tok_list, out, part_o, part_ml, counters, n_tokens, nh, nkv, page_size, \
                         max_blocks, splits, grid_splits, counter_tiles, scale, window, stream)
    switch (hd) {
        case 16: GO(16);
        case 32: GO(32);
        case 64: GO(64);
        case 96: GO(96);
        case 128: GO(128);
    }
#undef GO
    return VK_BAD_SHAPE;
}

}  // namespace vk
