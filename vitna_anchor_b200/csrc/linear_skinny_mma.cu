// The few-rows matrix product in bfloat16 on the tensor cores: out[M, N] = x[M, K] * W[N, K]^T, M <= 64,
// fused with RMSNorm before and with the rotation and cache write, SwiGLU or the residual sum after.
//
// Decoding streams every weight once and has almost no arithmetic, so what counts is how few
// instructions and how few dependent trips to memory a block needs.  One m16n8k16 instruction
// (weights as the 16-row operand, eight batch rows as the 8-column operand) replaces 64 float32
// multiply-adds.  A block owns eight "units" (pairs of weight rows, see below) and splits K over its
// warps; each warp issues all of its 16-byte weight loads before it uses any, the warps' partial sums
// meet in shared memory in a fixed order, and warp 0 (and others, for more than eight rows) finishes.
//
// Within a run of 32 columns lane (g, q) = (lane / 4, lane % 4) loads columns 8q .. 8q+7 of weight
// rows g and g+8 of the tile, and of batch row g: 16 contiguous bytes each.  The instruction's k index
// is a permutation of the memory column, the same for both operands, so the dot products are unchanged.
//
// Units, as in linear_skinny.cu: SAME / F32 / ACC rows (2u, 2u+1); SWIGLU rows (u, N/2 + u);
// ROPE the half-split pair (h*hd + j, h*hd + j + hd/2) of a q or k head, or two adjacent rows of v.
// A tile's rows 0..7 are the first rows of eight units and rows 8..15 their second rows, so a lane
// holds both values of a pair for two batch rows.
//
// Rounding points equal those of the separate kernels (values that would be stored in bfloat16 between
// two kernels are rounded to it here), and an output does not depend on M or on the other batch rows:
// the split of K over warps depends on K alone.
#include "common.cuh"

namespace vk {

enum { ME_SAME = 0, ME_F32 = 1, ME_ACC = 2, ME_SWIGLU = 3, ME_ROPE = 4 };
// Staged rows are 64 bytes (mod 128) apart, so that the eight lanes of a quarter warp (two rows, four 16-byte
// columns) read eight different 16-byte bank groups.

struct MmaParams {
    const void* x;               // NORM: float32 [*, K] rows of stride ldx; else bfloat16 [M, K] rows of stride ldx
    const int32_t* rows;         // NORM only, optional: input row of each of the M rows
    const float* norm_w;
    float eps;
    const __nv_bfloat16* w;      // [N, K]
    void* out;
    int M, N, K, ldx, kc, ks;    // kc: columns staged at a time (a multiple of 32 * ks); ks: warps = splits of K
    int xstride;                 // elements of bfloat16 between two staged rows
    int xoff;                    // where in a staged row its bfloat16 values begin (elements; not 0: behind the float32 values of the staged norm)
    int tpb;                     // most tiles of eight units a block works through (tile = blockIdx.x + i * gridDim.x)
    int depth;                   // streaming kernel: batches of weights in flight for every lane
    const int32_t* positions;
    const float* cos_t;
    const float* sin_t;
    const int32_t* slot;
    __nv_bfloat16* cache;
    int nh, nkv, hd, page_size;
};

__device__ __forceinline__ void mm_cp_async16(void* dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}

__device__ __forceinline__ float bf16_round(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }

__device__ __forceinline__ void mma_bf16(float* d, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

template <int EPI>
__device__ __forceinline__ void mma_unit_rows(const MmaParams& p, int u, int& r0, int& r1) {
    if (EPI == ME_SWIGLU) { r0 = u; r1 = p.N / 2 + u; }
    else if (EPI == ME_ROPE) {
        const int half = p.hd / 2, rot_units = (p.nh + p.nkv) * half;
        if (u < rot_units) { r0 = (u / half) * p.hd + u % half; r1 = r0 + half; }
        else { r0 = (p.nh + p.nkv) * p.hd + 2 * (u - rot_units); r1 = r0 + 1; }
    } else { r0 = 2 * u; r1 = 2 * u + 1; }
}

// One (unit, batch row) pair of sums -> its place.
template <int EPI>
__device__ __forceinline__ void mma_finish(const MmaParams& p, int u, int r0, int r1, bool has1, int m, float a0, float a1,
                                           bool pre, int pre_slot, float pre_cos, float pre_sin, const float* old) {
    typedef __nv_bfloat16 T;
    if (EPI == ME_SAME) {
        T* o = reinterpret_cast<T*>(p.out) + (size_t)m * p.N;
        o[r0] = __float2bfloat16_rn(a0);
        if (has1) o[r1] = __float2bfloat16_rn(a1);
    } else if (EPI == ME_F32) {
        float* o = reinterpret_cast<float*>(p.out) + (size_t)m * p.N;
        o[r0] = a0;
        if (has1) o[r1] = a1;
    } else if (EPI == ME_ACC) {
        float* o = reinterpret_cast<float*>(p.out) + (size_t)m * p.N;
        o[r0] = (pre ? old[0] : o[r0]) + a0;
        if (has1) o[r1] = (pre ? old[1] : o[r1]) + a1;
    } else if (EPI == ME_SWIGLU) {
        const float g = bf16_round(a0), up = bf16_round(a1);
        reinterpret_cast<T*>(p.out)[(size_t)m * (p.N / 2) + u] = __float2bfloat16_rn((g / (1.0f + expf(-g))) * up);
    } else {
        const int half = p.hd / 2, rot_units = (p.nh + p.nkv) * half;
        const int s = pre ? pre_slot : p.slot[m];
        const size_t page = s >= 0 ? (size_t)(s / p.page_size) : 0;
        const int off = s >= 0 ? s % p.page_size : 0;
        T* kbase = p.cache + page * 2 * p.nkv * p.page_size * p.hd;
        if (u < rot_units) {
            const int h = u / half, j = u % half;
            float c = pre_cos, sn = pre_sin;
            if (!pre) {
                const int pos = p.positions[m];
                c = p.cos_t[(size_t)pos * half + j];
                sn = p.sin_t[(size_t)pos * half + j];
            }
            const float a = bf16_round(a0), b = bf16_round(a1);
            const float ra = a * c - b * sn, rb = b * c + a * sn;
            if (h < p.nh) {
                T* qo = reinterpret_cast<T*>(p.out) + (size_t)m * p.nh * p.hd + h * p.hd;
                qo[j] = __float2bfloat16_rn(ra);
                qo[j + half] = __float2bfloat16_rn(rb);
            } else if (s >= 0) {
                T* dst = kbase + ((size_t)(h - p.nh) * p.page_size + off) * p.hd;
                dst[j] = __float2bfloat16_rn(ra);
                dst[j + half] = __float2bfloat16_rn(rb);
            }
        } else if (s >= 0) {
            const int col = 2 * (u - rot_units);
            T* vbase = kbase + (size_t)p.nkv * p.page_size * p.hd;
            T* dst = vbase + ((size_t)(col / p.hd) * p.page_size + off) * p.hd + col % p.hd;
            dst[0] = __float2bfloat16_rn(a0);
            dst[1] = __float2bfloat16_rn(a1);
        }
    }
}

// A row of up to 128 * NV float32 values straight from global memory into a warp's registers (all its 16-byte pieces
// on their way at once), normed there, left as bfloat16 in dst.  The sum of squares runs in the order of the staged
// path (a lane's pieces in ascending order, then the shuffle tree), so both give the same bits.
template <int NV>
__device__ __forceinline__ void norm_row_in_regs(const float* __restrict__ xr, const float* __restrict__ nw, int K, float eps,
                                                 __nv_bfloat16* dst, int lane) {
    float4 xv[NV];
#pragma unroll
    for (int j = 0; j < NV; j++) {
        const int k = lane * 4 + j * 128;
        if (k < K) xv[j] = *reinterpret_cast<const float4*>(xr + k);
    }
    float ss = 0.0f;
#pragma unroll
    for (int j = 0; j < NV; j++) {
        if (lane * 4 + j * 128 < K) {
            ss = fmaf(xv[j].x, xv[j].x, ss); ss = fmaf(xv[j].y, xv[j].y, ss); ss = fmaf(xv[j].z, xv[j].z, ss); ss = fmaf(xv[j].w, xv[j].w, ss);
        }
    }
    ss = warp_sum(ss);
    const float inv = 1.0f / sqrtf(ss / (float)K + eps);
#pragma unroll
    for (int j = 0; j < NV; j++) {
        const int k = lane * 4 + j * 128;
        if (k < K) {
            const float4 wv = __ldg(reinterpret_cast<const float4*>(nw + k));
            __nv_bfloat162 lo = __floats2bfloat162_rn((xv[j].x * inv) * wv.x, (xv[j].y * inv) * wv.y);
            __nv_bfloat162 hi = __floats2bfloat162_rn((xv[j].z * inv) * wv.z, (xv[j].w * inv) * wv.w);
            uint2 v;
            v.x = *reinterpret_cast<uint32_t*>(&lo);
            v.y = *reinterpret_cast<uint32_t*>(&hi);
            *reinterpret_cast<uint2*>(dst + k) = v;
        }
    }
}

// MG: groups of eight batch rows (1, 2, 4 or 8).  PIPE: the variant for long rows (two batches of loads a warp in flight).
// blockDim.x = 32 * ks.  Block (b, y) works on tiles b, b + gridDim.x, ... for batch rows y * MG*8 ...
template <int EPI, bool NORM, int MG, bool PIPE>
__global__ void __launch_bounds__(256, MG <= 4 ? 2 : 1) skinny_mma_kernel(const MmaParams p) {
    typedef __nv_bfloat16 T;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int xstride = p.xstride;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, q = lane & 3;
    const int K = p.K, ks = p.ks;
    const int m0 = blockIdx.y * (MG * 8);               // the block's batch rows: m0 .. m0 + MG*8 - 1
    // [MG*8][xstride] staged rows.  With the norm a row first holds the float32 input (4K bytes) and then, in its
    // first half, the normalised bfloat16 values; the norm's weights follow the rows.
    T* xs = reinterpret_cast<T*>(smem_raw);
    float* nw_s = reinterpret_cast<float*>(smem_raw + (size_t)MG * 8 * xstride * sizeof(T));
    float* red = nw_s + (NORM ? K : 0);                                        // [ks][MG][32][4]
    const int units = (EPI == ME_SWIGLU) ? p.N / 2 : (p.N + 1) / 2;

    // this lane's two weight rows: the first and second row of unit (tile*8 + g)
    int u = blockIdx.x * 8 + g;
    bool on = u < units;
    int r0 = 0, r1 = 0;
    if (on) mma_unit_rows<EPI>(p, u, r0, r1);
    bool has1 = on && r1 < p.N;
    const T* w0 = p.w + (size_t)r0 * K;
    const T* w1 = p.w + (size_t)(has1 ? r1 : r0) * K;

    // The first weights of this warp are asked for before anything that depends on the kernel before this one:
    // they are most of the wait of a decode layer, and they are nobody's output.
    constexpr int UN = 4;                               // runs of 32 columns in a batch: 8 loads of 16 bytes per lane
    uint4 wr[UN], ws[UN], wr2[PIPE ? UN : 1], ws2[PIPE ? UN : 1];
    {
        const int nblk0 = min(p.kc, K) / 32;
#pragma unroll
        for (int i = 0; i < UN; i++) {
            if (warp + i * ks < nblk0) {
                const int col = (warp + i * ks) * 32 + q * 8;
                wr[i] = __ldg(reinterpret_cast<const uint4*>(w0 + col));
                ws[i] = __ldg(reinterpret_cast<const uint4*>(w1 + col));
            }
        }
        if (PIPE) {
#pragma unroll
            for (int i = 0; i < UN; i++) {
                if (warp + (UN + i) * ks < nblk0) {
                    const int col = (warp + (UN + i) * ks) * 32 + q * 8;
                    wr2[i] = __ldg(reinterpret_cast<const uint4*>(w0 + col));
                    ws2[i] = __ldg(reinterpret_cast<const uint4*>(w1 + col));
                }
            }
        }
    }
    // With the fused norm, rows of up to NORM_REG columns never touch shared memory in float32: a warp takes a row
    // straight from global memory into registers (all its 16-byte pieces and the norm's weights on their way at once),
    // norms it there and leaves only the bfloat16 values.  Measured inside decode steps at K = 576, staging the rows in
    // float32 first (cp.async, a barrier, two passes over shared memory) took 2.8-3.2 of a kernel's 6.4 microseconds.
    // (Rows of up to 640 columns: with eight pieces a lane instead of five the kernel for K = 960 kept them in local
    // memory and a step at the 360M sizes took 1.27 instead of 1.20 ms.)
    constexpr int NORM_NV = 5, NORM_REG = 128 * NORM_NV;
    const bool norm_in_regs = NORM && K <= NORM_REG;
    int norm_src[2] = {0, 0};                           // the input rows of the warp's first two rows (an index array may name them)
    if (NORM && !norm_in_regs) {                        // the norm's weights, nobody's output either
        for (int k = tid * 4; k < K; k += blockDim.x * 4) mm_cp_async16(nw_s + k, p.norm_w + k);
    }
    if (norm_in_regs) {
#pragma unroll
        for (int e = 0; e < 2; e++) {
            const int m = m0 + warp + e * ks;
            norm_src[e] = (warp + e * ks < MG * 8 && m < p.M) ? (p.rows ? p.rows[m] : m) : 0;
        }
    }
    // what the first finishing pass of this lane needs besides the sums
    const int m_first = m0 + warp * 8 + 2 * q;          // rows m_first, m_first + 1 of row group `warp`
    int pre_slot[2] = {-1, -1}, pre_pos[2] = {0, 0};
    float pre_cos[2] = {1.0f, 1.0f}, pre_sin[2] = {0.0f, 0.0f};
    if (EPI == ME_ROPE && on && warp < MG) {
        const int half = p.hd / 2, rot_units = (p.nh + p.nkv) * half;
#pragma unroll
        for (int e = 0; e < 2; e++) {
            if (m_first + e < p.M) {
                pre_slot[e] = p.slot[m_first + e];
                pre_pos[e] = p.positions[m_first + e];
            }
        }
        if (u < rot_units) {
#pragma unroll
            for (int e = 0; e < 2; e++) {
                if (m_first + e < p.M) {
                    pre_cos[e] = p.cos_t[(size_t)pre_pos[e] * half + u % half];
                    pre_sin[e] = p.sin_t[(size_t)pre_pos[e] * half + u % half];
                }
            }
        }
    }
    dependency_wait();
    let_dependents_start();

    if (norm_in_regs) {
        const float* xg = reinterpret_cast<const float*>(p.x);
        int round = 0;
        for (int m = warp; m < MG * 8; m += ks, round++) {
            T* dst = xs + (size_t)m * xstride;
            if (m0 + m >= p.M) {
                for (int k = lane * 8; k < K; k += 256) *reinterpret_cast<uint4*>(dst + k) = make_uint4(0, 0, 0, 0);
                continue;
            }
            const int src = round < 2 ? norm_src[round] : (p.rows ? p.rows[m0 + m] : m0 + m);
            norm_row_in_regs<NORM_NV>(xg + (size_t)src * p.ldx, p.norm_w, K, p.eps, dst, lane);
        }
        __syncthreads();
    } else if (NORM) {
        // One trip to memory for all rows: every warp asks for its rows (float32) into their staging rows, then
        // norms them where they lie.  A row's sum of squares is one warp's, in a fixed order.
        for (int m = warp; m < MG * 8 && m0 + m < p.M; m += ks) {
            const int src = p.rows ? p.rows[m0 + m] : m0 + m;
            const float* xr = reinterpret_cast<const float*>(p.x) + (size_t)src * p.ldx;
            float* xf = reinterpret_cast<float*>(xs + (size_t)m * xstride);
            for (int k = lane * 4; k < K; k += 128) mm_cp_async16(xf + k, xr + k);
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    }
    // the values the residual sum adds to (read now, used at the end)
    float old[2][2] = {{0.0f, 0.0f}, {0.0f, 0.0f}};
    if (EPI == ME_ACC && on && warp < MG) {
#pragma unroll
        for (int e = 0; e < 2; e++) {
            if (m_first + e < p.M) {
                const float* o = reinterpret_cast<const float*>(p.out) + (size_t)(m_first + e) * p.N;
                old[e][0] = o[r0];
                if (has1) old[e][1] = o[r1];
            }
        }
    }
    if (NORM && !norm_in_regs) {
        asm volatile("cp.async.wait_group 0;" ::: "memory");
        __syncthreads();                                // the norm's weights came through all threads
        for (int m = warp; m < MG * 8; m += ks) {
            T* dst = xs + (size_t)m * xstride;
            if (m0 + m >= p.M) {
                for (int k = lane * 8; k < K; k += 256) *reinterpret_cast<uint4*>(dst + p.xoff + k) = make_uint4(0, 0, 0, 0);
                continue;
            }
            const float* xf = reinterpret_cast<const float*>(dst);
            float ss = 0.0f;
            for (int k = lane * 4; k < K; k += 128) {
                const float4 v = *reinterpret_cast<const float4*>(xf + k);
                ss = fmaf(v.x, v.x, ss); ss = fmaf(v.y, v.y, ss); ss = fmaf(v.z, v.z, ss); ss = fmaf(v.w, v.w, ss);
            }
            ss = warp_sum(ss);
            const float inv = 1.0f / sqrtf(ss / (float)K + p.eps);
            if (p.xoff) {
                // the bfloat16 values have a place of their own behind the row's float32 values: one pass, nothing to wait for
#pragma unroll 4
                for (int k = lane * 4; k < K; k += 128) {
                    const float4 xv = *reinterpret_cast<const float4*>(xf + k);
                    const float4 wv = *reinterpret_cast<const float4*>(nw_s + k);
                    __nv_bfloat162 lo = __floats2bfloat162_rn((xv.x * inv) * wv.x, (xv.y * inv) * wv.y);
                    __nv_bfloat162 hi = __floats2bfloat162_rn((xv.z * inv) * wv.z, (xv.w * inv) * wv.w);
                    uint2 v;
                    v.x = *reinterpret_cast<uint32_t*>(&lo);
                    v.y = *reinterpret_cast<uint32_t*>(&hi);
                    *reinterpret_cast<uint2*>(dst + p.xoff + k) = v;
                }
                continue;
            }
            // 128 columns at a time, upwards: the bfloat16 values of a run never reach float32 values not yet read
            for (int k0 = 0; k0 < K; k0 += 128) {
                const int k = k0 + lane * 4;
                float4 xv = make_float4(0.0f, 0.0f, 0.0f, 0.0f), wv = xv;
                if (k < K) {
                    xv = *reinterpret_cast<const float4*>(xf + k);
                    wv = *reinterpret_cast<const float4*>(nw_s + k);
                }
                __syncwarp();
                if (k < K) {
                    __nv_bfloat162 lo = __floats2bfloat162_rn((xv.x * inv) * wv.x, (xv.y * inv) * wv.y);
                    __nv_bfloat162 hi = __floats2bfloat162_rn((xv.z * inv) * wv.z, (xv.w * inv) * wv.w);
                    uint2 v;
                    v.x = *reinterpret_cast<uint32_t*>(&lo);
                    v.y = *reinterpret_cast<uint32_t*>(&hi);
                    *reinterpret_cast<uint2*>(dst + k) = v;
                }
                __syncwarp();
            }
        }
        __syncthreads();
    }

    const bool one_chunk = p.kc >= K;                   // then x is staged once for all of the block's tiles
  for (int it = 0; it < p.tpb; it++) {
    if (it > 0) {
        u += gridDim.x * 8;
        if ((u - g) >= units) break;                    // the same for the whole block
        on = u < units;
        r0 = r1 = 0;
        if (on) mma_unit_rows<EPI>(p, u, r0, r1);
        has1 = on && r1 < p.N;
        w0 = p.w + (size_t)r0 * K;
        w1 = p.w + (size_t)(has1 ? r1 : r0) * K;
    }
    float d[MG][4];
#pragma unroll
    for (int mg = 0; mg < MG; mg++) { d[mg][0] = d[mg][1] = d[mg][2] = d[mg][3] = 0.0f; }

    for (int kb = 0; kb < K; kb += p.kc) {
        const int kn = min(p.kc, K - kb);               // a multiple of 32
        if (!NORM && (it == 0 || !one_chunk)) {
            __syncthreads();                            // the previous chunk has been read
            // stage rows 0..M-1 (rows up to MG*8 are zero) of columns kb .. kb+kn
            // (cp.async: all of a lane's pieces are on their way at once; through registers, four at a time, a long row
            // took several trips to the second-level cache)
            for (int m = warp; m < MG * 8; m += ks) {
                T* dst = xs + (size_t)m * xstride;
                if (m0 + m >= p.M) {
                    for (int k = lane * 8; k < kn; k += 256) *reinterpret_cast<uint4*>(dst + k) = make_uint4(0, 0, 0, 0);
                } else {
                    const T* xr = reinterpret_cast<const T*>(p.x) + (size_t)(m0 + m) * p.ldx + kb;
                    for (int k = lane * 8; k < kn; k += 256) mm_cp_async16(dst + k, xr + k);
                }
            }
            asm volatile("cp.async.commit_group;" ::: "memory");
            asm volatile("cp.async.wait_group 0;" ::: "memory");
            __syncthreads();
        }
        // this warp's share of the chunk: the runs of 32 columns whose index is warp modulo ks.  A chunk starts
        // at a multiple of 32 * ks, so which warp adds a run, and in which order, depends on K alone.
        const int nblk = kn / 32;
        const bool fresh = it == 0 && kb == 0;          // then the first loads are already on their way
        auto load_batch = [&](uint4* r, uint4* t, int b) {
#pragma unroll
            for (int i = 0; i < UN; i++) {
                if (b + i * ks < nblk) {
                    const int col = kb + (b + i * ks) * 32 + q * 8;
                    r[i] = __ldg(reinterpret_cast<const uint4*>(w0 + col));
                    t[i] = __ldg(reinterpret_cast<const uint4*>(w1 + col));
                }
            }
        };
        auto use_batch = [&](const uint4* r, const uint4* t, int b) {
#pragma unroll
            for (int i = 0; i < UN; i++) {
                if (b + i * ks < nblk) {
#pragma unroll
                    for (int mg = 0; mg < MG; mg++) {
                        const uint4 xv = *reinterpret_cast<const uint4*>(xs + (size_t)(mg * 8 + g) * xstride + p.xoff + (b + i * ks) * 32 + q * 8);
                        mma_bf16(d[mg], r[i].x, t[i].x, r[i].y, t[i].y, xv.x, xv.y);
                        mma_bf16(d[mg], r[i].z, t[i].z, r[i].w, t[i].w, xv.z, xv.w);
                    }
                }
            }
        };
        if (PIPE) {
            // long rows: two batches of loads are in flight, one being used while the next travels
            int b = warp;
            if (!fresh) load_batch(wr, ws, b);
            bool have2 = fresh;
            while (b < nblk) {
                int b2 = b + UN * ks;
                if (b2 < nblk && !have2) load_batch(wr2, ws2, b2);
                have2 = false;
                use_batch(wr, ws, b);
                b = b2;
                if (b >= nblk) break;
                b2 = b + UN * ks;
                if (b2 < nblk) load_batch(wr, ws, b2);
                use_batch(wr2, ws2, b);
                b = b2;
            }
        } else {
            for (int b = warp; b < nblk; b += UN * ks) {
                if (!fresh || b != warp) load_batch(wr, ws, b);
                use_batch(wr, ws, b);
            }
        }
    }
    // partial sums of the warps meet in shared memory; warp w then finishes the row groups w, w+ks, ...
#pragma unroll
    for (int mg = 0; mg < MG; mg++)
        *reinterpret_cast<float4*>(red + (((size_t)warp * MG + mg) * 32 + lane) * 4) = make_float4(d[mg][0], d[mg][1], d[mg][2], d[mg][3]);
    __syncthreads();
    for (int mg = warp; mg < MG; mg += ks) {
        float4 s = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        for (int w = 0; w < ks; w++) {
            const float4 v = *reinterpret_cast<const float4*>(red + (((size_t)w * MG + mg) * 32 + lane) * 4);
            s.x += v.x; s.y += v.y; s.z += v.z; s.w += v.w;
        }
        if (!on) continue;
        // lane (g, q): unit u; batch rows mg*8 + 2q and + 1; s.x, s.y are row r0's sums, s.z, s.w row r1's
        const int m = m0 + mg * 8 + 2 * q;
        const bool first = it == 0 && mg == warp;       // this pass has its extras in registers already
        if (m < p.M) mma_finish<EPI>(p, u, r0, r1, has1, m, s.x, s.z, first, pre_slot[0], pre_cos[0], pre_sin[0], old[0]);
        if (m + 1 < p.M) mma_finish<EPI>(p, u, r0, r1, has1, m + 1, s.y, s.w, first, pre_slot[1], pre_cos[1], pre_sin[1], old[1]);
    }
    __syncthreads();                                    // the partial sums have been read: the next tile may write its own
  }
}


// ---------------------------------------------------------------------------------------------------------------
// The streaming variant, for long rows and for launches in which a block works through several tiles.
//
// The kernel above asks for a tile's weights (two batches of a warp's share before the wait on the kernel before it),
// waits, multiplies, lets the warps' sums meet and only then asks for the next tile: between two tiles a block has
// nothing on its way, and a row too long for two batches costs a trip to memory after the wait.  Measured alone over
// weights larger than the second-level cache, this one reads 67 MB (gate and up at the 1.7B sizes, eight rows) in 14.7
// microseconds (4.6 TB/s) and the 201 MB of that model's output matrix at 5.6 TB/s (a library reduction over 1 GiB
// reads at 5.9), the kernel above in 19.9 and at 4.5.  Here a lane
// keeps `depth` batches of its own weights (four runs of 32 columns, two rows: 128 bytes) on their way into a ring in
// shared memory that only this lane reads back (cp.async; consecutive lanes write consecutive 16 bytes), across
// tiles and across the meeting of the warps.  One block a multiprocessor; the ring takes what shared memory the
// staged rows leave.  Which warp adds which run, and in which order, is as above, so the sums are the same bits.
// ---------------------------------------------------------------------------------------------------------------
constexpr int ST_UN = 4, ST_ROUND = 4;      // runs of 32 columns in a batch; tiles whose sums a warp keeps before the warps meet

__device__ __forceinline__ void st_wait_pending(int n) {        // until at most n of the lane's latest batches are on their way
    switch (n) {
        case 0: asm volatile("cp.async.wait_group 0;" ::: "memory"); break;
        case 1: asm volatile("cp.async.wait_group 1;" ::: "memory"); break;
        case 2: asm volatile("cp.async.wait_group 2;" ::: "memory"); break;
        case 3: asm volatile("cp.async.wait_group 3;" ::: "memory"); break;
        case 4: asm volatile("cp.async.wait_group 4;" ::: "memory"); break;
        case 5: asm volatile("cp.async.wait_group 5;" ::: "memory"); break;
        case 6: asm volatile("cp.async.wait_group 6;" ::: "memory"); break;
        default: asm volatile("cp.async.wait_group 7;" ::: "memory"); break;
    }
}

template <int EPI, bool NORM, int MG>
__global__ void __launch_bounds__(256, 1) skinny_stream_kernel(const MmaParams p) {
    typedef __nv_bfloat16 T;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int xstride = p.xstride;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nth = blockDim.x;
    const int g = lane >> 2, q = lane & 3;
    const int K = p.K, ks = p.ks, kc = p.kc, depth = p.depth;
    const int m0 = blockIdx.y * (MG * 8);
    T* xs = reinterpret_cast<T*>(smem_raw);
    float* nw_s = reinterpret_cast<float*>(smem_raw + (size_t)MG * 8 * xstride * sizeof(T));
    float* red = nw_s + (NORM ? K : 0);                                        // [ks][MG][32][4]
    uint4* ring = reinterpret_cast<uint4*>(red + (size_t)ks * ST_ROUND * MG * 32 * 4);    // [depth][ST_UN][2][nth]
    const int units = (EPI == ME_SWIGLU) ? p.N / 2 : (p.N + 1) / 2;
    const int total_tiles = (units + 7) / 8;
    const int n_my = (int)blockIdx.x < total_tiles ? (total_tiles - 1 - (int)blockIdx.x) / (int)gridDim.x + 1 : 0;

    auto tile_rows = [&](int it, int& u, bool& on, int& r0, int& r1, bool& has1) {
        u = ((int)blockIdx.x + it * (int)gridDim.x) * 8 + g;
        on = u < units;
        r0 = r1 = 0;
        if (on) mma_unit_rows<EPI>(p, u, r0, r1);
        has1 = on && r1 < p.N;
    };
    // ---- the side that asks: batch after batch in the order the other side uses them ----------------------------
    int l_it = 0, l_kb = 0, l_b = warp;
    const T *lw0 = p.w, *lw1 = p.w;
    auto loader_tile = [&]() {
        int u, r0, r1; bool on, has1;
        tile_rows(l_it, u, on, r0, r1, has1);
        lw0 = p.w + (size_t)r0 * K;
        lw1 = p.w + (size_t)(has1 ? r1 : r0) * K;
    };
    if (n_my > 0) loader_tile();
    auto ask = [&](int slot) {
        if (l_it < n_my) {
            const int nblk = min(kc, K - l_kb) / 32;
#pragma unroll
            for (int i = 0; i < ST_UN; i++) {
                const int bb = l_b + i * ks;
                if (bb < nblk) {
                    const int col = l_kb + bb * 32 + q * 8;
                    uint4* dst = ring + ((size_t)(slot * ST_UN + i) * 2) * nth + tid;
                    mm_cp_async16(dst, lw0 + col);
                    mm_cp_async16(dst + nth, lw1 + col);
                }
            }
            l_b += ST_UN * ks;
            if (l_b >= nblk) {                          // a chunk is at least one batch for every warp, be it empty
                l_b = warp;
                l_kb += kc;
                if (l_kb >= K) {
                    l_kb = 0;
                    l_it++;
                    if (l_it < n_my) loader_tile();
                }
            }
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    // weights are nobody's output: the first batches are on their way before the kernel before this one has finished
    for (int sl = 0; sl < depth; sl++) ask(sl);
    constexpr int ST_NORM_NV = 16;                      // rows of up to 2,048 columns are normed in registers (one block a multiprocessor: registers to spare)
    const bool norm_in_regs = NORM && K <= 128 * ST_NORM_NV;
    if (NORM && !norm_in_regs) {
        for (int k = tid * 4; k < K; k += nth * 4) mm_cp_async16(nw_s + k, p.norm_w + k);
    }
    dependency_wait();
    let_dependents_start();

    if (norm_in_regs) {
        for (int m = warp; m < MG * 8; m += ks) {
            T* dst = xs + (size_t)m * xstride;
            if (m0 + m >= p.M) {
                for (int k = lane * 8; k < K; k += 256) *reinterpret_cast<uint4*>(dst + k) = make_uint4(0, 0, 0, 0);
                continue;
            }
            const int src = p.rows ? p.rows[m0 + m] : m0 + m;
            norm_row_in_regs<ST_NORM_NV>(reinterpret_cast<const float*>(p.x) + (size_t)src * p.ldx, p.norm_w, K, p.eps, dst, lane);
        }
        __syncthreads();
    } else if (NORM) {                                  // as above: the rows in float32, normed where they lie
        for (int m = warp; m < MG * 8 && m0 + m < p.M; m += ks) {
            const int src = p.rows ? p.rows[m0 + m] : m0 + m;
            const float* xr = reinterpret_cast<const float*>(p.x) + (size_t)src * p.ldx;
            float* xf = reinterpret_cast<float*>(xs + (size_t)m * xstride);
            for (int k = lane * 4; k < K; k += 128) mm_cp_async16(xf + k, xr + k);
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
        asm volatile("cp.async.wait_group 0;" ::: "memory");       // the rows came last; the first batches are here too
        __syncthreads();
        for (int m = warp; m < MG * 8; m += ks) {
            T* dst = xs + (size_t)m * xstride;
            if (m0 + m >= p.M) {
                for (int k = lane * 8; k < K; k += 256) *reinterpret_cast<uint4*>(dst + k) = make_uint4(0, 0, 0, 0);
                continue;
            }
            const float* xf = reinterpret_cast<const float*>(dst);
            float ss = 0.0f;
            for (int k = lane * 4; k < K; k += 128) {
                const float4 v = *reinterpret_cast<const float4*>(xf + k);
                ss = fmaf(v.x, v.x, ss); ss = fmaf(v.y, v.y, ss); ss = fmaf(v.z, v.z, ss); ss = fmaf(v.w, v.w, ss);
            }
            ss = warp_sum(ss);
            const float inv = 1.0f / sqrtf(ss / (float)K + p.eps);
            for (int k0 = 0; k0 < K; k0 += 128) {
                const int k = k0 + lane * 4;
                float4 xv = make_float4(0.0f, 0.0f, 0.0f, 0.0f), wv = xv;
                if (k < K) {
                    xv = *reinterpret_cast<const float4*>(xf + k);
                    wv = *reinterpret_cast<const float4*>(nw_s + k);
                }
                __syncwarp();
                if (k < K) {
                    __nv_bfloat162 lo = __floats2bfloat162_rn((xv.x * inv) * wv.x, (xv.y * inv) * wv.y);
                    __nv_bfloat162 hi = __floats2bfloat162_rn((xv.z * inv) * wv.z, (xv.w * inv) * wv.w);
                    uint2 v;
                    v.x = *reinterpret_cast<uint32_t*>(&lo);
                    v.y = *reinterpret_cast<uint32_t*>(&hi);
                    *reinterpret_cast<uint2*>(dst + k) = v;
                }
                __syncwarp();
            }
        }
        __syncthreads();
    }

    // ---- the side that multiplies -------------------------------------------------------------------------------
    // ST_ROUND tiles a round: a warp keeps the sums of the round's tiles in registers, and the warps meet once a round
    // (one pair of barriers for four tiles, and up to four warps finish a tile each) instead of once a tile: with
    // short rows the meeting was most of a tile's time.
    const bool one_chunk = kc >= K;
    int slot = 0;
    for (int it0 = 0; it0 < n_my; it0 += ST_ROUND) {
        float d[ST_ROUND][MG][4];
#pragma unroll
        for (int tt = 0; tt < ST_ROUND; tt++) {
#pragma unroll
            for (int mg = 0; mg < MG; mg++) { d[tt][mg][0] = d[tt][mg][1] = d[tt][mg][2] = d[tt][mg][3] = 0.0f; }
        }
#pragma unroll
        for (int tt = 0; tt < ST_ROUND; tt++) {
            const int it = it0 + tt;
            if (it >= n_my) break;                      // the same for the whole block
            for (int kb = 0; kb < K; kb += kc) {
                const int kn = min(kc, K - kb);
                if (!NORM && (it == 0 || !one_chunk)) {
                    __syncthreads();                    // the chunk before has been read
                    for (int m = warp; m < MG * 8; m += ks) {
                        T* dst = xs + (size_t)m * xstride;
                        if (m0 + m >= p.M) {
                            for (int k = lane * 8; k < kn; k += 256) *reinterpret_cast<uint4*>(dst + k) = make_uint4(0, 0, 0, 0);
                        } else {
                            const T* xr = reinterpret_cast<const T*>(p.x) + (size_t)(m0 + m) * p.ldx + kb;
                            for (int k = lane * 8; k < kn; k += 256) mm_cp_async16(dst + k, xr + k);
                        }
                    }
                    // the rows came last: the batches of weights asked for before them are here too, and the count of
                    // batches on their way starts again from none
                    asm volatile("cp.async.commit_group;" ::: "memory");
                    asm volatile("cp.async.wait_group 0;" ::: "memory");
                    __syncthreads();
                }
                const int nblk = kn / 32;
                int b = warp;
                do {
                    st_wait_pending(depth - 1);         // the oldest batch on its way is the one used now
#pragma unroll
                    for (int i = 0; i < ST_UN; i++) {
                        const int bb = b + i * ks;
                        if (bb < nblk) {
                            const uint4* src = ring + ((size_t)(slot * ST_UN + i) * 2) * nth + tid;
                            const uint4 r = src[0], t = src[nth];
#pragma unroll
                            for (int mg = 0; mg < MG; mg++) {
                                const uint4 xv = *reinterpret_cast<const uint4*>(xs + (size_t)(mg * 8 + g) * xstride + bb * 32 + q * 8);
                                mma_bf16(d[tt][mg], r.x, t.x, r.y, t.y, xv.x, xv.y);
                                mma_bf16(d[tt][mg], r.z, t.z, r.w, t.w, xv.z, xv.w);
                            }
                        }
                    }
                    ask(slot);                          // the place just read takes the batch `depth` further on
                    slot = slot + 1 == depth ? 0 : slot + 1;
                    b += ST_UN * ks;
                } while (b < nblk);
            }
        }
        // the warps' sums of the round's tiles meet; warp w then finishes the pairs (tile, row group) w, w + ks, ...
#pragma unroll
        for (int tt = 0; tt < ST_ROUND; tt++) {
#pragma unroll
            for (int mg = 0; mg < MG; mg++)
                *reinterpret_cast<float4*>(red + ((((size_t)warp * ST_ROUND + tt) * MG + mg) * 32 + lane) * 4) =
                    make_float4(d[tt][mg][0], d[tt][mg][1], d[tt][mg][2], d[tt][mg][3]);
        }
        __syncthreads();
        for (int idx = warp; idx < ST_ROUND * MG; idx += ks) {
            const int tt = idx / MG, mg = idx % MG, it = it0 + tt;
            if (it >= n_my) continue;
            float4 s = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            for (int w = 0; w < ks; w++) {
                const float4 v = *reinterpret_cast<const float4*>(red + ((((size_t)w * ST_ROUND + tt) * MG + mg) * 32 + lane) * 4);
                s.x += v.x; s.y += v.y; s.z += v.z; s.w += v.w;
            }
            int u, r0, r1; bool on, has1;
            tile_rows(it, u, on, r0, r1, has1);
            if (!on) continue;
            const int m = m0 + mg * 8 + 2 * q;
            if (m < p.M) mma_finish<EPI>(p, u, r0, r1, has1, m, s.x, s.z, false, 0, 1.0f, 0.0f, nullptr);
            if (m + 1 < p.M) mma_finish<EPI>(p, u, r0, r1, has1, m + 1, s.y, s.w, false, 0, 1.0f, 0.0f, nullptr);
        }
        __syncthreads();
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
}

// 0: never the streaming kernel, 1: whenever its sizes fit, 2 (default): long rows or several tiles a block (see launch_stream).
static int g_stream_mode = -1;
static int stream_mode() {
    if (g_stream_mode < 0) {
        const char* e = getenv("VITNA_SKINNY_STREAM");
        g_stream_mode = e ? atoi(e) : 2;
    }
    return g_stream_mode;
}

// Launches the streaming kernel if it should and can take the product; returns -1 if not.
template <int EPI, bool NORM>
static int launch_stream(MmaParams p, int mg, int ks, cudaStream_t stream) {
    if (mg > 2 || stream_mode() == 0) return -1;
    const int units = (EPI == ME_SWIGLU) ? p.N / 2 : (p.N + 1) / 2;
    const int tiles = (units + 7) / 8;
    const int ychunks = (p.M + 8 * mg - 1) / (8 * mg);
    const int per_chunk = 148 / ychunks > 0 ? 148 / ychunks : 1;
    const int blocks = tiles < per_chunk ? tiles : per_chunk;
    // Measured inside decode steps (batch 8, milliseconds a step with and without): it wins where the rows are long
    // (K >= 2,048: the kernel above has two batches of a warp's weights on their way before the wait, and a third costs a
    // trip after it; 360M 1.135 -> 1.029, 1.7B 1.850 -> 1.814) and where a block walks through two tiles or more (the
    // output matrix).  With short rows and few tiles the kernel above, two blocks a multiprocessor and room beside
    // the kernels before and after it, is the faster one (135M with K >= 1,024 streamed: 0.659 against 0.645), and so
    // it is when the batch rows are split over blocks.
    if (stream_mode() == 2 && !(ychunks == 1 && (p.K >= 2048 || tiles >= 2 * 148))) return -1;
    const int rows = mg * 8, nth = 32 * ks;
    const size_t stage = (size_t)ST_UN * 2 * 16 * nth;                  // a batch of every lane
    const size_t red = (size_t)ks * ST_ROUND * mg * 32 * 4 * sizeof(float);
    const size_t budget = 224 * 1024;
    int kc = p.K;
    size_t stride_bytes, fixed;
    if (NORM) {
        stride_bytes = (size_t)4 * p.K + 64;
        fixed = rows * stride_bytes + (size_t)4 * p.K + red;
        if (fixed + 2 * stage > budget) return -1;
    } else {
        // the rows take at most what leaves the ring four batches: columns in multiples of 32 * ks
        const size_t room = budget - red - 4 * stage;
        const int fit = (int)(((room / rows - 64) / 2) / (32 * ks)) * (32 * ks);
        if (fit <= 0) return -1;
        if (kc > fit) kc = fit;
        stride_bytes = (size_t)2 * kc + ((2 * kc) % 128 == 64 ? 0 : 64);
        fixed = rows * stride_bytes + red;
    }
    int depth = (int)((budget - fixed) / stage);
    if (depth > 8) depth = 8;
    if (depth < 2) return -1;
    p.ks = ks;
    p.kc = kc;
    p.xstride = (int)(stride_bytes / 2);
    p.depth = depth;
    p.tpb = (tiles + blocks - 1) / blocks;
    const size_t smem = fixed + depth * stage;
#define LAUNCH_ST(MGV)                                                                                                      \
    {                                                                                                                       \
        auto kern = skinny_stream_kernel<EPI, NORM, MGV>;                                                                   \
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);                 \
        if (e != cudaSuccess) return (int)e;                                                                                \
        const int rc = launch_dependent(kern, dim3(blocks, ychunks), dim3(nth), smem, stream, p);                           \
        if (rc != 0) return rc;                                                                                             \
    }
    if (mg == 1) LAUNCH_ST(1) else LAUNCH_ST(2)
#undef LAUNCH_ST
    return launch_status();
}

template <int EPI, bool NORM>
static int launch_mma(MmaParams p, cudaStream_t stream) {
    const int units = (EPI == ME_SWIGLU) ? p.N / 2 : (p.N + 1) / 2;
    const int tiles = (units + 7) / 8;
    // Batch rows a block: all of them (in groups of eight), unless the weights make too few tiles to fill the
    // machine; then the rows are split over blocks too, and the weights come several times, from the second-level cache.
    // Small weights (up to 16 MB) never get more than 16 rows a block: re-reading them from the second-level cache
    // is cheap, and 16 rows are few enough for the norm to be fused.
    int mg = p.M <= 8 ? 1 : p.M <= 16 ? 2 : p.M <= 32 ? 4 : 8;
    if (mg > 2 && (size_t)p.N * p.K * 2 <= ((size_t)16 << 20)) mg = 2;
    while (mg > 1 && tiles * ((p.M + 8 * mg - 1) / (8 * mg)) < 120) mg /= 2;
    const int ychunks = (p.M + 8 * mg - 1) / (8 * mg);
    const int nblk = p.K / 32;
    // warps that split K (K alone decides): between 4 and 8 if that divides the runs of 32 columns evenly,
    // else as many as leave a warp at least two runs
    int ks = 0;
    for (int cand = 8; cand >= 4 && !ks; cand--)
        if (nblk % cand == 0) ks = cand;
    if (!ks) { ks = 8; while (ks > 1 && nblk / ks < 2) ks--; }
    p.ks = ks;
    {
        const int rc = launch_stream<EPI, NORM>(p, mg, ks, stream);
        if (rc >= 0) return rc;
    }
    // columns staged at a time: all of K if the rows fit in 160 KB, else the largest multiple of 32*ks that does.
    // With the norm a row is staged whole, in float32.
    const int rows = mg * 8;
    int kc = p.K;
    size_t stride_bytes;
    p.xoff = 0;
    if (NORM) {
        stride_bytes = (size_t)4 * p.K + 64;            // K is a multiple of 32: 4K is a multiple of 128
        // Rows too long to be normed in registers get, where two blocks still share a multiprocessor, a place of their own
        // for the bfloat16 values behind the float32 ones (the norm then needs no care about what it overwrites).
        const size_t wide = (size_t)6 * p.K + ((6 * p.K) % 128 == 64 ? 0 : 64);
        if (p.K > 640 && rows * wide + (size_t)4 * p.K + (size_t)ks * mg * 32 * 4 * sizeof(float) + 1024 <= 113 * 1024) {
            stride_bytes = wide;
            p.xoff = 2 * p.K;
        }
    } else {
        const int fit = ((163840 / rows - 64) / 2) / (32 * ks) * (32 * ks);
        if (kc > fit) kc = fit;
        if (kc <= 0) return VK_TOO_LARGE;
        stride_bytes = (size_t)2 * kc + ((2 * kc) % 128 == 64 ? 0 : 64);
    }
    p.kc = kc;
    p.xstride = (int)(stride_bytes / 2);
    const size_t smem = (size_t)rows * stride_bytes + (NORM ? (size_t)4 * p.K : 0) + (size_t)ks * mg * 32 * 4 * sizeof(float);
    if (smem > 220 * 1024) return VK_TOO_LARGE;
    // a block stages x (and computes the norm) for itself, so there are no more blocks than are resident at once
    // (two a multiprocessor, one if the staged rows are large); each takes every gridDim.x-th tile
    // (the row chunks share them)
    const int resident = 148 * (smem + 1024 <= 113 * 1024 ? 2 : 1);
    const int per_chunk = resident / ychunks > 0 ? resident / ychunks : 1;
    const int blocks = tiles < per_chunk ? tiles : per_chunk;
    p.tpb = (tiles + blocks - 1) / blocks;
    const bool pipe = nblk / ks > 4;                    // more than one batch of four runs a warp
#define LAUNCH(MGV)                                                                                                         \
    if (pipe) LAUNCH2(MGV, true) else LAUNCH2(MGV, false)
#define LAUNCH2(MGV, PV)                                                                                                    \
    {                                                                                                                       \
        auto kern = skinny_mma_kernel<EPI, NORM, MGV, PV>;                                                                  \
        if (smem > 48 * 1024) {                                                                                             \
            cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);             \
            if (e != cudaSuccess) return (int)e;                                                                            \
        }                                                                                                                   \
        const int rc = launch_dependent(kern, dim3(blocks, ychunks), dim3(32 * ks), smem, stream, p);                                \
        if (rc != 0) return rc;                                                                                             \
    }
    if (mg == 1) LAUNCH(1) else if (mg == 2) LAUNCH(2) else if (mg == 4) LAUNCH(4) else LAUNCH(8)
#undef LAUNCH
#undef LAUNCH2
    return launch_status();
}

template <bool NORM>
static int mma_dispatch(int epi, const MmaParams& p, cudaStream_t stream) {
    switch (epi) {
        case ME_SAME: return launch_mma<ME_SAME, NORM>(p, stream);
        case ME_F32: return launch_mma<ME_F32, NORM>(p, stream);
        case ME_ACC: return launch_mma<ME_ACC, NORM>(p, stream);
        case ME_SWIGLU: return launch_mma<ME_SWIGLU, NORM>(p, stream);
        case ME_ROPE: return launch_mma<ME_ROPE, NORM>(p, stream);
    }
    return VK_BAD_SHAPE;
}

}  // namespace vk

using namespace vk;

// Which launches the streaming kernel takes (see stream_mode); returns the mode that was in force.
VK_API int vk_set_skinny_stream(int mode) {
    const int was = stream_mode();
    if (mode >= 0 && mode <= 2) g_stream_mode = mode;
    return was;
}

// The bfloat16 few-rows product on tensor cores.  Arguments as vk_linear_skinny; in addition K must be a
// multiple of 32, and with the fused norm x's rows must be 16-byte aligned (ldx a multiple of 4).
VK_API int vk_linear_skinny_mma(const void* x, const int32_t* rows, const float* norm_w, float eps, const void* w, void* out,
                                int M, int N, int K, int ldx, int epi, const int32_t* positions, const float* cos_t,
                                const float* sin_t, const int32_t* slot, void* cache, int nh, int nkv, int hd, int page_size,
                                cudaStream_t stream) {
    if (M <= 0 || N <= 0) return VK_OK;
    if (K <= 0 || ldx < K || epi < 0 || epi > 4 || K % 32 != 0) return VK_BAD_SHAPE;
    if (M > 64) return VK_TOO_LARGE;
    if (((uintptr_t)w % 16) || ((uintptr_t)x % 16)) return VK_BAD_ALIGNMENT;
    if (norm_w ? (ldx % 4 != 0 || ((uintptr_t)norm_w % 16)) : (ldx % 8 != 0)) return VK_BAD_ALIGNMENT;
    if (epi == ME_SWIGLU && (N % 2)) return VK_BAD_SHAPE;
    if (epi == ME_ROPE) {
        if (nh <= 0 || nkv <= 0 || hd <= 0 || (hd % 2) || page_size <= 0 || N != (nh + 2 * nkv) * hd || !positions || !cos_t || !sin_t ||
            !slot || !cache)
            return VK_BAD_SHAPE;
    }
    MmaParams p{x, rows, norm_w, eps, (const __nv_bfloat16*)w, out, M, N, K, ldx, 0, 0, 0, 0, 1, 0, positions, cos_t, sin_t, slot,
                (__nv_bfloat16*)cache, nh, nkv, hd, page_size};
    return norm_w ? mma_dispatch<true>(epi, p, stream) : mma_dispatch<false>(epi, p, stream);
}
