// Causal attention of prompt portions over the paged cache, in bfloat16 on the tensor cores.
//
// A block takes 64 consecutive tokens of one request (a "query tile") and one query head.  It has two
// groups of four warps; a warp owns 16 query rows, and the two groups share the key tiles between them
// (group 0 the even ones counted from the first, group 1 the odd ones), which halves the longest chain
// of the causal triangle; their running (maximum, sum, output) meet once at the end, group 0 first.
// Keys and values of the request are read from its pages in tiles of 64 positions whose boundaries are
// multiples of 64 in absolute position, so the order of a row's sums does not depend on how the prompt
// was cut into steps.  Scores S = Q K^T (mma m16n8k16,
// float32 accumulation) are scaled after the sum, masked (a query at position p sees keys
// max(0, p - window + 1) .. p), and folded into a running maximum, sum and output in float32
// (the softmax of engine/src/model.c:932-956, computed tile by tile).  The tensor cores take P in
// bfloat16: each probability goes in as a high and a low bfloat16 part (p = hi + lo to about 2^-17), so
// that P V matches the float32 probabilities of the decode kernel instead of differing from it by a
// rounding of every p.  Head sizes: multiples of 16 up to 128 that are instantiated below.
//
// tiles [n_tiles][4] int32: first token (flat index), rows (1..64), position of the first token, segment.
#include "common.cuh"

namespace vk {

constexpr int PF_BM = 64, PF_BN = 64, PF_THREADS = 256, PF_GROUP = 128;

__device__ __forceinline__ void cp_async16(void* dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__device__ __forceinline__ void ldsm_x4(uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3, const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"((uint32_t)__cvta_generic_to_shared(p)));
}
__device__ __forceinline__ void ldsm_x4_trans(uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3, const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"((uint32_t)__cvta_generic_to_shared(p)));
}
__device__ __forceinline__ void mma16816(float* d, const uint32_t* a, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// 2^x by the special-function unit (about 2 units in the last place of float32; 2^-inf = 0).
__device__ __forceinline__ float ex2_approx(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

template <int HD>
__global__ void __launch_bounds__(PF_THREADS, 2) attention_prefill_kernel(
    const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ cache, const int32_t* __restrict__ block_tables,
    const int32_t* __restrict__ tiles, __nv_bfloat16* __restrict__ out, int nh, int nkv, int page_size, int max_blocks, float scale,
    int window) {
    typedef __nv_bfloat16 T;
    constexpr int LD = HD + 8;                      // padded row: 16-byte shifts keep ldmatrix free of bank conflicts
    constexpr int KSTEPS = HD / 16;                 // k-steps of Q K^T
    constexpr int DBLK = HD / 8;                    // 8-wide blocks of the output
    extern __shared__ __align__(16) unsigned char smem_raw[];
    T* sq = reinterpret_cast<T*>(smem_raw);         // [64][LD]
    const int grp = threadIdx.x / PF_GROUP;         // which half of the key tiles
    T* sk = sq + PF_BM * LD + grp * 4 * PF_BN * LD; // this group's [2][64][LD]
    T* sv = sk + 2 * PF_BN * LD;                    // this group's [2][64][LD]

    const int tile = gridDim.x - 1 - blockIdx.x;    // later tiles of a prompt have more keys: start them first
    const int h = blockIdx.y;
    const int kvh = h / (nh / nkv);
    const int tok0 = tiles[tile * 4 + 0], rows = tiles[tile * 4 + 1], pos0 = tiles[tile * 4 + 2], seg = tiles[tile * 4 + 3];
    const int tid = threadIdx.x % PF_GROUP, warp = tid >> 5, lane = tid & 31;      // within the group
    const int g = lane >> 2, qd = lane & 3;
    const int32_t* bt = block_tables + (size_t)seg * max_blocks;
    const size_t page_stride = (size_t)2 * nkv * page_size * HD;
    const size_t v_off = (size_t)nkv * page_size * HD;

    const float scale_log2 = scale * 1.4426950408889634f;
    const int last_pos = pos0 + rows - 1;
    const int lo_first = (window > 0 && pos0 - window + 1 > 0) ? pos0 - window + 1 : 0;     // lowest key any row needs
    const int kt0 = lo_first / PF_BN, kt1 = last_pos / PF_BN;                               // key tiles kt0 .. kt1

    // ---- loads ------------------------------------------------------------------------------------
    constexpr int CHUNKS = HD / 8;                  // 16-byte chunks per row
    auto load_q = [&]() {
        for (int i = threadIdx.x; i < PF_BM * CHUNKS; i += PF_THREADS) {
            const int r = i / CHUNKS, c = i % CHUNKS;
            T* dst = sq + r * LD + c * 8;
            if (r < rows) cp_async16(dst, q + ((size_t)(tok0 + r) * nh + h) * HD + c * 8);
            else *reinterpret_cast<uint4*>(dst) = make_uint4(0, 0, 0, 0);
        }
    };
    auto load_kv = [&](int kt, int buf) {
        T* dk = sk + buf * PF_BN * LD;
        T* dv = sv + buf * PF_BN * LD;
        for (int i = tid; i < PF_BN * CHUNKS; i += PF_GROUP) {
            const int r = i / CHUNKS, c = i % CHUNKS;
            const int key = kt * PF_BN + r;
            if (key <= last_pos && key >= lo_first) {
                const T* src = cache + (size_t)bt[key / page_size] * page_stride + ((size_t)kvh * page_size + key % page_size) * HD + c * 8;
                cp_async16(dk + r * LD + c * 8, src);
                cp_async16(dv + r * LD + c * 8, src + v_off);
            } else {                                // never read as a key (masked), but keep the values finite
                *reinterpret_cast<uint4*>(dk + r * LD + c * 8) = make_uint4(0, 0, 0, 0);
                *reinterpret_cast<uint4*>(dv + r * LD + c * 8) = make_uint4(0, 0, 0, 0);
            }
        }
    };

    auto group_sync = [&]() { asm volatile("bar.sync %0, %1;" ::"r"(1 + grp), "n"(PF_GROUP) : "memory"); };
    const int kfirst = kt0 + grp;                   // this group's key tiles: kfirst, kfirst + 2, ...
    dependency_wait();                              // q and the cache come from the kernels before this one
    let_dependents_start();
    load_q();
    if (kfirst <= kt1) load_kv(kfirst, 0);
    cp_async_commit();

    // per-thread state: rows g and g+8 of this warp's 16 query rows
    float o[DBLK][4];
#pragma unroll
    for (int i = 0; i < DBLK; i++) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.0f; }
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.0f, 0.0f};
    uint32_t qf[KSTEPS][4];
    const int row_a = warp * 16 + g, row_b = row_a + 8;          // rows within the tile
    const int pos_a = pos0 + row_a, pos_b = pos0 + row_b;
    const int lo_a = (window > 0 && pos_a - window + 1 > 0) ? pos_a - window + 1 : 0;
    const int lo_b = (window > 0 && pos_b - window + 1 > 0) ? pos_b - window + 1 : 0;

    cp_async_wait<0>();
    __syncthreads();                                // q (loaded by both groups) and each group's first tile
    for (int kt = kfirst; kt <= kt1; kt += 2) {
        const int buf = ((kt - kfirst) >> 1) & 1;
        if (kt + 2 <= kt1) load_kv(kt + 2, buf ^ 1);
        cp_async_commit();
        if (kt != kfirst) {
            cp_async_wait<1>();
            group_sync();
        }
        if (kt == kfirst) {
            // this warp's Q fragments, once
#pragma unroll
            for (int ks = 0; ks < KSTEPS; ks++) {
                const T* p = sq + (warp * 16 + (lane & 15)) * LD + ks * 16 + (lane >> 4) * 8;
                ldsm_x4(qf[ks][0], qf[ks][1], qf[ks][2], qf[ks][3], p);
            }
        }
        const T* k_s = sk + buf * PF_BN * LD;
        const T* v_s = sv + buf * PF_BN * LD;

        // a warp whose 16 rows all lie before this key tile, or whose windows all lie after it, has nothing to add
        const int warp_last = pos0 + warp * 16 + 15;
        const int warp_lo = (window > 0 && pos0 + warp * 16 - window + 1 > 0) ? pos0 + warp * 16 - window + 1 : 0;
        const bool any = kt * PF_BN <= warp_last && kt * PF_BN + PF_BN - 1 >= warp_lo;
        if (any) {
            // ---- S = Q K^T for 64 keys: 8 blocks of 8 keys ----------------------------------------------
            float s[8][4];
#pragma unroll
            for (int nb = 0; nb < 8; nb++) { s[nb][0] = s[nb][1] = s[nb][2] = s[nb][3] = 0.0f; }
#pragma unroll
            for (int ks = 0; ks < KSTEPS; ks++) {
#pragma unroll
                for (int nb2 = 0; nb2 < 4; nb2++) {         // two key blocks per ldmatrix.x4
                    uint32_t b0, b1, b2, b3;
                    const T* p = k_s + (nb2 * 16 + (lane & 7) + ((lane >> 4) << 3)) * LD + ks * 16 + ((lane >> 3) & 1) * 8;
                    ldsm_x4(b0, b1, b2, b3, p);
                    mma16816(s[nb2 * 2], qf[ks], b0, b1);
                    mma16816(s[nb2 * 2 + 1], qf[ks], b2, b3);
                }
            }
            // ---- scale, mask, running softmax (in base 2: exp(x) = exp2(x * log2 e), folded into the scale) ----------
            float mx[2] = {-INFINITY, -INFINITY};
            // every key of the tile visible to every row of this warp: no mask to apply
            const int warp_lo_last = (window > 0 && pos0 + warp * 16 + 15 - window + 1 > 0) ? pos0 + warp * 16 + 15 - window + 1 : 0;
            const bool all_visible = kt * PF_BN + PF_BN - 1 <= pos0 + warp * 16 && kt * PF_BN >= warp_lo_last;
            // the running maximum is kept of the raw scores (the scale is positive); the scale and log2 e go into
            // the exponent's multiply-add.  Only tiles that touch the diagonal or a window's edge need the mask.
            if (all_visible) {
#pragma unroll
                for (int nb = 0; nb < 8; nb++) {
                    mx[0] = fmaxf(mx[0], fmaxf(s[nb][0], s[nb][1]));
                    mx[1] = fmaxf(mx[1], fmaxf(s[nb][2], s[nb][3]));
                }
            } else {
#pragma unroll
                for (int nb = 0; nb < 8; nb++) {
#pragma unroll
                    for (int e = 0; e < 4; e++) {
                        const int key = kt * PF_BN + nb * 8 + qd * 2 + (e & 1);
                        const bool second = e >= 2;
                        const int pos = second ? pos_b : pos_a, lo = second ? lo_b : lo_a;
                        const float v = (key <= pos && key >= lo) ? s[nb][e] : -INFINITY;
                        s[nb][e] = v;
                        mx[second] = fmaxf(mx[second], v);
                    }
                }
            }
#pragma unroll
            for (int r = 0; r < 2; r++) {
                mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
                mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
            }
            float corr[2], m_new[2];      // m_new: minus the reference maximum times scale * log2 e
#pragma unroll
            for (int r = 0; r < 2; r++) {
                const float mm = fmaxf(m_run[r], mx[r]);
                // a row with no key yet (all masked so far) keeps m = -inf: use 0 as the reference so that exp gives 0
                const float ref = mm == -INFINITY ? 0.0f : mm;
                corr[r] = ex2_approx((m_run[r] - ref) * scale_log2);     // 2^(-inf) = 0 on the first tile with keys
                m_run[r] = mm;
                m_new[r] = -ref * scale_log2;
            }
            float rs[2] = {0.0f, 0.0f};
            uint32_t pf[4][4], pl[4][4];                 // P as A fragments, high and low parts: 4 k-steps of 16 keys
#pragma unroll
            for (int nb = 0; nb < 8; nb++) {
                const float p0 = ex2_approx(fmaf(s[nb][0], scale_log2, m_new[0])), p1 = ex2_approx(fmaf(s[nb][1], scale_log2, m_new[0]));
                const float p2 = ex2_approx(fmaf(s[nb][2], scale_log2, m_new[1])), p3 = ex2_approx(fmaf(s[nb][3], scale_log2, m_new[1]));
                rs[0] += p0 + p1;
                rs[1] += p2 + p3;
                const uint32_t h01 = pack_bf16(p0, p1), h23 = pack_bf16(p2, p3);
                pf[nb >> 1][(nb & 1) * 2] = h01;
                pf[nb >> 1][(nb & 1) * 2 + 1] = h23;
                pl[nb >> 1][(nb & 1) * 2] = pack_bf16(p0 - __uint_as_float(h01 << 16), p1 - __uint_as_float(h01 & 0xffff0000u));
                pl[nb >> 1][(nb & 1) * 2 + 1] = pack_bf16(p2 - __uint_as_float(h23 << 16), p3 - __uint_as_float(h23 & 0xffff0000u));
            }
#pragma unroll
            for (int r = 0; r < 2; r++) {
                rs[r] += __shfl_xor_sync(0xffffffffu, rs[r], 1);
                rs[r] += __shfl_xor_sync(0xffffffffu, rs[r], 2);
                l_run[r] = l_run[r] * corr[r] + rs[r];
            }
#pragma unroll
            for (int i = 0; i < DBLK; i++) { o[i][0] *= corr[0]; o[i][1] *= corr[0]; o[i][2] *= corr[1]; o[i][3] *= corr[1]; }
            // ---- O += P V: k = keys (4 steps of 16), n = head dimensions (blocks of 8) ---------------------------
#pragma unroll
            for (int kk = 0; kk < 4; kk++) {
#pragma unroll
                for (int db2 = 0; db2 < DBLK / 2; db2++) {   // two blocks of 8 dimensions per ldmatrix.x4.trans
                    uint32_t b0, b1, b2, b3;
                    const T* p = v_s + (kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * LD + db2 * 16 + (lane >> 4) * 8;
                    ldsm_x4_trans(b0, b1, b2, b3, p);
                    mma16816(o[db2 * 2], pf[kk], b0, b1);
                    mma16816(o[db2 * 2 + 1], pf[kk], b2, b3);
                    mma16816(o[db2 * 2], pl[kk], b0, b1);
                    mma16816(o[db2 * 2 + 1], pl[kk], b2, b3);
                }
            }
        }
        group_sync();           // the buffer is free for the load after next
    }
    cp_async_wait<0>();

    // ---- the two groups' running results meet: group 1 hands over, group 0 folds it in after its own -----------
    __syncthreads();            // every key tile is consumed: the tile buffers are free
    float* hand = reinterpret_cast<float*>(sq + PF_BM * LD + 4 * PF_BN * LD);     // group 1's buffers, [128][DBLK*4 + 4]
    constexpr int HW = DBLK * 4 + 4;
    if (grp == 1) {
        float* mine = hand + tid * HW;
        mine[0] = m_run[0]; mine[1] = m_run[1]; mine[2] = l_run[0]; mine[3] = l_run[1];
#pragma unroll
        for (int i = 0; i < DBLK; i++) { mine[4 + i * 4] = o[i][0]; mine[5 + i * 4] = o[i][1]; mine[6 + i * 4] = o[i][2]; mine[7 + i * 4] = o[i][3]; }
    }
    __syncthreads();
    if (grp == 1) return;
    {
        const float* other = hand + tid * HW;
#pragma unroll
        for (int r = 0; r < 2; r++) {
            const float m1 = other[r], l1 = other[2 + r];
            const float mm = fmaxf(m_run[r], m1);
            const float ref = mm == -INFINITY ? 0.0f : mm;
            const float c0 = ex2_approx((m_run[r] - ref) * scale_log2), c1 = ex2_approx((m1 - ref) * scale_log2);
            l_run[r] = l_run[r] * c0 + l1 * c1;
#pragma unroll
            for (int i = 0; i < DBLK; i++) {
                o[i][2 * r] = o[i][2 * r] * c0 + other[4 + i * 4 + 2 * r] * c1;
                o[i][2 * r + 1] = o[i][2 * r + 1] * c0 + other[4 + i * 4 + 2 * r + 1] * c1;
            }
        }
    }

    // ---- normalise and store ---------------------------------------------------------------------------
    const float inv_a = l_run[0] > 0.0f ? 1.0f / l_run[0] : 0.0f, inv_b = l_run[1] > 0.0f ? 1.0f / l_run[1] : 0.0f;
#pragma unroll
    for (int i = 0; i < DBLK; i++) {
        const int d = i * 8 + qd * 2;
        if (row_a < rows)
            *reinterpret_cast<uint32_t*>(out + ((size_t)(tok0 + row_a) * nh + h) * HD + d) = pack_bf16(o[i][0] * inv_a, o[i][1] * inv_a);
        if (row_b < rows)
            *reinterpret_cast<uint32_t*>(out + ((size_t)(tok0 + row_b) * nh + h) * HD + d) = pack_bf16(o[i][2] * inv_b, o[i][3] * inv_b);
    }
}

template <int HD>
static int launch_prefill(const void* q, const void* cache, const int32_t* bt, const int32_t* tiles, void* out, int n_tiles, int nh,
                          int nkv, int page_size, int max_blocks, float scale, int window, cudaStream_t stream) {
    constexpr int LD = HD + 8;
    const size_t smem = (size_t)(PF_BM + 8 * PF_BN) * LD * 2;
    auto kern = attention_prefill_kernel<HD>;
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
    }
    dim3 grid(n_tiles, nh);
    return launch_plain(kern, grid, dim3(PF_THREADS), smem, stream, (const __nv_bfloat16*)q, (const __nv_bfloat16*)cache, bt, tiles,
                            (__nv_bfloat16*)out, nh, nkv, page_size, max_blocks, scale, window);
}

}  // namespace vk

using namespace vk;

// bfloat16 only.  q, out [all tokens, nh*hd]; cache: one layer [pages][2][nkv][page_size][hd];
// tiles [n_tiles][4]: first token, rows (1..64), position of the first token, segment (row of block_tables).
VK_API int vk_attention_prefill(const void* q, const void* cache, const int32_t* block_tables, const int32_t* tiles, void* out,
                                int n_tiles, int nh, int nkv, int hd, int page_size, int max_blocks, float scale, int window,
                                cudaStream_t stream) {
    if (n_tiles <= 0) return VK_OK;
    if (nh <= 0 || nkv <= 0 || nh % nkv != 0 || page_size <= 0 || max_blocks <= 0 || window < 0) return VK_BAD_SHAPE;
    if (nh > 65535) return VK_TOO_LARGE;
    if (((uintptr_t)q % 16) || ((uintptr_t)cache % 16) || ((uintptr_t)out % 4)) return VK_BAD_ALIGNMENT;
#define GO(HD) return launch_prefill<HD>(q, cache, block_tables, tiles, out, n_tiles, nh, nkv, page_size, max_blocks, scale, window, stream)
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
