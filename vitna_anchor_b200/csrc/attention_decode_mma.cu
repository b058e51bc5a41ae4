// Split-key decode attention in bfloat16 with the scores and p*v on the tensor cores.
//
// Same decomposition and scratch as attention_decode.cu: grid = (splits of 256 keys at absolute positions,
// kv-head tiles, tokens); each block leaves an unnormalised partial and the last block of a
// (token, kv-head tile) combines them in split order.  What differs is the arithmetic of a block: the
// query heads that share a key-value head (up to 16 a block) are the 16 rows of an m16n8k16 product.
//
// Within a block every warp works alone on 32 of the split's keys, with no barrier until the end:
//
//   copy      the warp's keys and values into shared memory with cp.async, whole lines at a time; the queries go
//             straight from global memory into the registers of the 16-row operand
//   scores    S[16 heads x 32 keys] = Q K^T
//   softmax   against the warp's own row maxima, float32
//   p * v     the probabilities go from the score registers straight into the 16-row operand, as a high and a
//             low bfloat16 part (p = hi + lo to about 2^-17, see attention_prefill.cu)
//   meet      the eight warps' unnormalised parts are weighted by exp(own maximum - row maximum) and added in
//             warp order
//
// A tile of at most eight heads (every group of this architecture's published sizes) turns the products over: the
// keys are the 16 rows and the heads the 8 columns, S^T = K Q^T and O^T = V^T P^T, with the probabilities
// transposed in registers (movmatrix) on their way into the 8-column operand.  Half the products and
// exponentials; the parts that the warp leaves have the same layout either way.
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

// One unit of work: a token, a tile of up to 16 query heads that share a key-value head, a split of 256 keys.
struct DmItem {
    bool active;
    int zi, t, y, split, kvh, h0, gt, pos, lo, first_split, last_split, n_active, k0, nkeys;
    const int32_t* bt;
};

struct DmArgs {
    const __nv_bfloat16* q;
    const __nv_bfloat16* cache;
    const int32_t* block_tables;
    const int32_t* token_seg;
    const int32_t* positions;
    const int32_t* tok_list;
    __nv_bfloat16* out;
    float* part_o;
    float* part_ml;
    int* counters;
    int nh, nkv, page_size, page_shift, max_blocks, max_splits, counter_tiles;   // page_shift: log2 of page_size, or -1
    float scale;
    int window;
};

__device__ __forceinline__ DmItem dm_item(const DmArgs& a, int zi, int y, int split) {
    DmItem it;
    const int g = a.nh / a.nkv;
    const int tiles_per_kv = (g + DM_ROWS - 1) / DM_ROWS;
    it.zi = zi; it.y = y; it.split = split;
    it.kvh = y / tiles_per_kv;
    it.h0 = it.kvh * g + (y % tiles_per_kv) * DM_ROWS;
    it.gt = min(DM_ROWS, it.kvh * g + g - it.h0);
    it.t = a.tok_list ? a.tok_list[zi] : zi;
    it.pos = a.positions[it.t];
    it.lo = (a.window > 0 && it.pos - a.window + 1 > 0) ? it.pos - a.window + 1 : 0;
    it.first_split = it.lo / DM_SPLIT;
    it.last_split = min(it.pos / DM_SPLIT, (int)gridDim.x - 1);     // see attention_decode.cu: only launched blocks are counted
    it.active = split >= it.first_split && split <= it.last_split;
    it.n_active = it.last_split - it.first_split + 1;
    it.k0 = split * DM_SPLIT;
    it.nkeys = min(DM_SPLIT, it.pos - it.k0 + 1);
    it.bt = a.block_tables + (size_t)a.token_seg[it.t] * a.max_blocks;
    return it;
}

__device__ __forceinline__ void dm_ldsm_x4_trans(uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3, const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"((uint32_t)__cvta_generic_to_shared(p)));
}
// 2^x in one instruction of the special-function unit: scores and maxima are kept in base 2 (the scale carries log2 e).
__device__ __forceinline__ float dm_ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ uint32_t dm_pack(float x, float y) {
    __nv_bfloat162 v = __floats2bfloat162_rn(x, y);
    return *reinterpret_cast<uint32_t*>(&v);
}

// Warp w asks for keys and values 32w .. 32w+31 of the split with cp.async: consecutive lanes take consecutive
// 16-byte pieces, so a request covers whole 128-byte lines (the keys of a page lie one after the other).  The
// pages of the warp's keys are read from the block table in one trip (lane p reads the p-th of them) and handed
// round by shuffle: a trip to memory per copy was a third of the block's time.  Rows that do not count are zeroed
// (never counted, p = 0, but 0 * garbage must not be NaN).  No commit.
//
// The key and value at the token's own position are left out: they are what the kernel before this one writes, and
// this copy runs before the wait for that kernel (dm_copy_own brings them afterwards).  Every earlier key of the
// request was written by an earlier step.  Returns the page of the token's own position (to every lane).
template <int HD>
__device__ __forceinline__ int dm_copy_warp(const DmArgs& a, const DmItem& it, __nv_bfloat16* sk, __nv_bfloat16* sv) {
    typedef __nv_bfloat16 T;
    constexpr int LD = HD + 8, CH = HD / 8;             // CH pieces of 16 bytes a row
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const size_t page_stride = (size_t)2 * a.nkv * a.page_size * HD;
    const size_t v_off = (size_t)a.nkv * a.page_size * HD;
    const int wk0 = it.k0 + warp * 32;                  // the warp's first key
    const int pg0 = a.page_shift >= 0 ? wk0 >> a.page_shift : wk0 / a.page_size;
    const int pg_last = a.page_shift >= 0 ? it.pos >> a.page_shift : it.pos / a.page_size;     // the request has pages up to here
    const int my_page = pg0 + lane <= pg_last ? it.bt[pg0 + lane] : 0;        // at most 32 pages hold 32 keys
#pragma unroll
    for (int i = 0; i < CH; i++) {
        const int c = i * 32 + lane;
        const int kl = warp * 32 + c / CH, part = c % CH;
        const int key = it.k0 + kl;
        const int pg = a.page_shift >= 0 ? key >> a.page_shift : key / a.page_size;
        const int page = __shfl_sync(0xffffffffu, my_page, pg - pg0);
        T* dk = sk + kl * LD + part * 8;
        T* dv = sv + kl * LD + part * 8;
        if (kl < it.nkeys && key >= it.lo) {
            if (key < it.pos) {
                const int off = key - pg * a.page_size;
                const T* kr = a.cache + (size_t)page * page_stride + ((size_t)it.kvh * a.page_size + off) * HD + part * 8;
                dm_cp_async16(dk, kr);
                dm_cp_async16(dv, kr + v_off);
            }
        } else {
            *reinterpret_cast<uint4*>(dk) = make_uint4(0, 0, 0, 0);
            *reinterpret_cast<uint4*>(dv) = make_uint4(0, 0, 0, 0);
        }
    }
    return __shfl_sync(0xffffffffu, my_page, min(max(pg_last - pg0, 0), 31));
}

// The key and value at the token's own position, for the warp whose 32 keys hold it: lanes 0 .. HD/8-1 copy a piece each.
template <int HD>
__device__ __forceinline__ void dm_copy_own(const DmArgs& a, const DmItem& it, int own_page, __nv_bfloat16* sk, __nv_bfloat16* sv) {
    typedef __nv_bfloat16 T;
    constexpr int LD = HD + 8, CH = HD / 8;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int kl = it.pos - it.k0;
    if (kl < warp * 32 || kl >= warp * 32 + 32 || lane >= CH) return;
    const int pg = a.page_shift >= 0 ? it.pos >> a.page_shift : it.pos / a.page_size;
    const int off = it.pos - pg * a.page_size;
    const T* kr = a.cache + (size_t)own_page * 2 * a.nkv * a.page_size * HD + ((size_t)it.kvh * a.page_size + off) * HD + lane * 8;
    dm_cp_async16(sk + kl * LD + lane * 8, kr);
    dm_cp_async16(sv + kl * LD + lane * 8, kr + (size_t)a.nkv * a.page_size * HD);
}

// The queries of the item's heads as the 16-row operand of m16n8k16, straight from global memory into registers
// (rows beyond the item's heads are zero): lane (gq, qd) holds rows gq and gq+8, columns 2qd, 2qd+1 and +8 of each k-step.
template <int HD>
__device__ __forceinline__ void dm_load_q(const DmArgs& a, const DmItem& it, uint32_t (*qf)[4]) {
    const int lane = threadIdx.x & 31, gq = lane >> 2, qd = lane & 3;
    const __nv_bfloat16* r0 = a.q + ((size_t)it.t * a.nh + it.h0 + gq) * HD + 2 * qd;
    const __nv_bfloat16* r1 = r0 + (size_t)8 * HD;
    const bool on0 = gq < it.gt, on1 = gq + 8 < it.gt;
#pragma unroll
    for (int ks = 0; ks < HD / 16; ks++) {
        qf[ks][0] = on0 ? *reinterpret_cast<const uint32_t*>(r0 + ks * 16) : 0u;
        qf[ks][1] = on1 ? *reinterpret_cast<const uint32_t*>(r1 + ks * 16) : 0u;
        qf[ks][2] = on0 ? *reinterpret_cast<const uint32_t*>(r0 + ks * 16 + 8) : 0u;
        qf[ks][3] = on1 ? *reinterpret_cast<const uint32_t*>(r1 + ks * 16 + 8) : 0u;
    }
}

__device__ __forceinline__ uint32_t dm_movmatrix_trans(uint32_t x) {
    uint32_t y;
    asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(y) : "r"(x));
    return y;
}

// A warp's 32 keys for a tile of AT MOST EIGHT query heads, with the keys (not the heads) as the 16 rows of the products:
// S^T[16 keys x 8 heads] = K Q^T (the keys' rows come with ldmatrix, the queries straight from global memory as the
// 8-column operand) and O^T[16 dims x 8 heads] = V^T P^T (V^T by a transposing ldmatrix; the probabilities go from
// the score registers through movmatrix into the 8-column operand, again as a high and a low bfloat16 part).  Half the
// products and half the exponentials of the routine with the heads as rows, which wastes thirteen of sixteen rows on
// a group of three heads.  Leaves the warp's maxima and sums in wml and its unnormalised output [head][HD] in wo.
template <int HD>
__device__ __forceinline__ void dm_warp_few_heads(const DmArgs& a, const DmItem& it, const __nv_bfloat16* sk, const __nv_bfloat16* sv,
                                                  float* wml, float* wo, float scale_log2) {
    typedef __nv_bfloat16 T;
    constexpr int LD = HD + 8, KSTEPS = HD / 16, HB = HD / 16;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, gq = lane >> 2, qd = lane & 3;
    const int wk0 = it.k0 + warp * 32, pos = it.pos, lo = it.lo, gt = it.gt;
    // the queries as the 8-column operand: lane (gq, qd) holds head gq, dims 2qd, 2qd+1 and +8 of each k-step
    uint32_t qb[KSTEPS][2];
    {
        const T* qr = a.q + ((size_t)it.t * a.nh + it.h0 + gq) * HD + 2 * qd;
        const bool on = gq < gt;
#pragma unroll
        for (int ks = 0; ks < KSTEPS; ks++) {
            qb[ks][0] = on ? *reinterpret_cast<const uint32_t*>(qr + ks * 16) : 0u;
            qb[ks][1] = on ? *reinterpret_cast<const uint32_t*>(qr + ks * 16 + 8) : 0u;
        }
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    __syncwarp();
    // ---- scores: two blocks of 16 keys; lane (gq, qd) gets keys gq and gq+8 of a block for heads 2qd, 2qd+1 ----------
    float s[2][4];
#pragma unroll
    for (int kb = 0; kb < 2; kb++) {
        s[kb][0] = s[kb][1] = s[kb][2] = s[kb][3] = 0.0f;
#pragma unroll
        for (int ks = 0; ks < KSTEPS; ks++) {
            uint32_t af[4];
            dm_ldsm_x4(af[0], af[1], af[2], af[3], sk + (warp * 32 + kb * 16 + (lane & 15)) * LD + ks * 16 + (lane >> 4) * 8);
            dm_mma(s[kb], af, qb[ks][0], qb[ks][1]);
        }
    }
    const bool edge = wk0 + 31 > pos || wk0 < lo;
    float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int kb = 0; kb < 2; kb++) {
#pragma unroll
        for (int e = 0; e < 4; e++) {
            float v = s[kb][e] * scale_log2;
            if (edge) {
                const int kk = wk0 + kb * 16 + gq + (e >> 1) * 8;
                if (!(kk <= pos && kk >= lo)) v = -INFINITY;
            }
            s[kb][e] = v;
            mx[e & 1] = fmaxf(mx[e & 1], v);
        }
    }
#pragma unroll
    for (int h = 0; h < 2; h++) {                       // over the eight lanes that hold the head's other keys
        mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 4));
        mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 8));
        mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 16));
    }
    float rs[2] = {0.0f, 0.0f};
    uint32_t ph[2][2], pl[2][2];                        // the 8-column operand of the two blocks of 16 keys, high and low parts
#pragma unroll
    for (int kb = 0; kb < 2; kb++) {
#pragma unroll
        for (int half = 0; half < 2; half++) {          // keys gq (0) and gq+8 (1) of the block
            const float p0 = dm_ex2(s[kb][2 * half] - mx[0]), p1 = dm_ex2(s[kb][2 * half + 1] - mx[1]);
            rs[0] += p0;
            rs[1] += p1;
            const __nv_bfloat162 hv = __floats2bfloat162_rn(p0, p1);
            const uint32_t hi = *reinterpret_cast<const uint32_t*>(&hv);
            const uint32_t lw = dm_pack(p0 - __bfloat162float(hv.x), p1 - __bfloat162float(hv.y));
            // [key][heads 2qd, 2qd+1] -> [head][keys 2qd, 2qd+1]: what the 8-column operand wants
            ph[kb][half] = dm_movmatrix_trans(hi);
            pl[kb][half] = dm_movmatrix_trans(lw);
        }
    }
#pragma unroll
    for (int h = 0; h < 2; h++) {
        rs[h] += __shfl_xor_sync(0xffffffffu, rs[h], 4);
        rs[h] += __shfl_xor_sync(0xffffffffu, rs[h], 8);
        rs[h] += __shfl_xor_sync(0xffffffffu, rs[h], 16);
    }
    if (gq == 0) {
        *reinterpret_cast<float2*>(wml + (warp * DM_ROWS + 2 * qd) * 2) = make_float2(mx[0], rs[0]);
        *reinterpret_cast<float2*>(wml + (warp * DM_ROWS + 2 * qd + 1) * 2) = make_float2(mx[1], rs[1]);
    }
    // ---- O^T = V^T P^T: blocks of 16 dims; lane (gq, qd) gets dims gq and gq+8 of a block for heads 2qd, 2qd+1 ----------
    float o[HB][4];
#pragma unroll
    for (int hb = 0; hb < HB; hb++) { o[hb][0] = o[hb][1] = o[hb][2] = o[hb][3] = 0.0f; }
#pragma unroll
    for (int kb = 0; kb < 2; kb++) {
#pragma unroll
        for (int hb = 0; hb < HB; hb++) {
            uint32_t af[4];
            dm_ldsm_x4_trans(af[0], af[1], af[2], af[3],
                             sv + (warp * 32 + kb * 16 + (lane & 7) + ((lane >> 4) << 3)) * LD + hb * 16 + ((lane >> 3) & 1) * 8);
            dm_mma(o[hb], af, ph[kb][0], ph[kb][1]);
            dm_mma(o[hb], af, pl[kb][0], pl[kb][1]);
        }
    }
    __syncwarp();                                       // every lane is past its reads of the warp's keys
#pragma unroll
    for (int hb = 0; hb < HB; hb++) {
        const int d = hb * 16 + gq;
#pragma unroll
        for (int e = 0; e < 2; e++) {
            const int head = 2 * qd + e;
            if (head < gt) {
                wo[head * HD + d] = o[hb][e];
                wo[head * HD + d + 8] = o[hb][2 + e];
            }
        }
    }
}

// Shared memory of a block: keys [256][HD+8], values [256][HD+8] and the warps' maxima and sums [8][16][2].  A warp's unnormalised output [16][HD] float32 lies over its own 32 keys,
// dead once it has its scores.  74 KB at HD = 64: three blocks a multiprocessor.
template <int HD> struct DmSmem {
    static constexpr int LD = HD + 8;
    static constexpr size_t KV_BYTES = (size_t)2 * DM_SPLIT * LD * 2;
    static constexpr size_t BYTES = KV_BYTES + 8 * DM_ROWS * 2 * 4;
};

// Every warp works alone on its 32 keys: copy, scores, softmax against its own maximum, p * v with the
// probabilities going from the score registers straight into the 16-row operand (as a high and a low bfloat16
// part, p = hi + lo to about 2^-17).  Only then do the warps meet: their eight parts are weighted and added in
// warp order, and the block leaves its partial (or, for a single split, the result).
template <int HD>
__global__ void __launch_bounds__(DM_THREADS, HD <= 64 ? 3 : 1) attention_decode_mma_kernel(const DmArgs a) {
    typedef __nv_bfloat16 T;
    typedef DmSmem<HD> L;
    constexpr int LD = HD + 8, KSTEPS = HD / 16, DBLK = HD / 8;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    T* sk = reinterpret_cast<T*>(smem_raw);                 // [256][LD]
    T* sv = sk + DM_SPLIT * LD;                             // [256][LD]
    float* wml = reinterpret_cast<float*>(smem_raw + L::KV_BYTES);   // [8 warps][16 rows][2]: maximum, sum
    __shared__ int is_last;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int gq = lane >> 2, qd = lane & 3;

    const DmItem it = dm_item(a, blockIdx.z, blockIdx.y, blockIdx.x);      // from the step's metadata, which no kernel writes
    if (!it.active) return;
    const int nh = a.nh, max_splits = a.max_splits;
    const int zi = it.zi, t = it.t, split = it.split, h0 = it.h0, gt = it.gt, pos = it.pos, lo = it.lo, k0 = it.k0;
    const int first_split = it.first_split, n_active = it.n_active;
    const float scale_log2 = a.scale * 1.4426950408889634f;         // scores, maxima and the partials' maxima are kept in base 2
    // keys of this warp: wk0 .. wk0+31; the warp has work if one of them counts
    const int wk0 = k0 + warp * 32;
    const bool warp_on = wk0 <= pos && wk0 + 31 >= lo;
    // The keys and values of earlier steps are asked for before the wait: they are most of what a block reads,
    // and the kernel before this one writes the token's own key and value only.
    int own_page = 0;
    if (warp_on) own_page = dm_copy_warp<HD>(a, it, sk, sv);
    dependency_wait();                          // q and the token's own key and value come from the kernel before this one
    let_dependents_start();

    float* wo = reinterpret_cast<float*>(sk + warp * 32 * LD);       // [16][HD], over the warp's own keys
    if (warp_on && gt <= 8) {
        dm_copy_own<HD>(a, it, own_page, sk, sv);
        asm volatile("cp.async.commit_group;" ::: "memory");
        dm_warp_few_heads<HD>(a, it, sk, sv, wml, wo, scale_log2);
    } else if (warp_on) {
        dm_copy_own<HD>(a, it, own_page, sk, sv);
        asm volatile("cp.async.commit_group;" ::: "memory");
        uint32_t qf[KSTEPS][4];
        dm_load_q<HD>(a, it, qf);
        asm volatile("cp.async.wait_group 0;" ::: "memory");
        __syncwarp();

        // ---- scores of the warp's 32 keys: four blocks of 8 keys --------------------------------------------
        float s[4][4];
#pragma unroll
        for (int nb = 0; nb < 4; nb++) { s[nb][0] = s[nb][1] = s[nb][2] = s[nb][3] = 0.0f; }
#pragma unroll
        for (int ks = 0; ks < KSTEPS; ks++) {
#pragma unroll
            for (int nb2 = 0; nb2 < 2; nb2++) {
                uint32_t b0, b1, b2, b3;
                dm_ldsm_x4(b0, b1, b2, b3, sk + (warp * 32 + nb2 * 16 + (lane & 7) + ((lane >> 4) << 3)) * LD + ks * 16 + ((lane >> 3) & 1) * 8);
                dm_mma(s[nb2 * 2], qf[ks], b0, b1);
                dm_mma(s[nb2 * 2 + 1], qf[ks], b2, b3);
            }
        }
        // scale (base 2) and, in a warp whose keys touch the position or the window's edge, mask; rows gq and gq+8
        // (heads), keys wk0 + nb*8 + 2*qd + {0,1}
        float mx[2] = {-INFINITY, -INFINITY};
        const bool edge = wk0 + 31 > pos || wk0 < lo;
#pragma unroll
        for (int nb = 0; nb < 4; nb++) {
#pragma unroll
            for (int e = 0; e < 4; e++) {
                float v = s[nb][e] * scale_log2;
                if (edge) {
                    const int kk = wk0 + nb * 8 + qd * 2 + (e & 1);
                    if (!(kk <= pos && kk >= lo)) v = -INFINITY;
                }
                s[nb][e] = v;
                mx[e >> 1] = fmaxf(mx[e >> 1], v);
            }
        }
        float rs[2] = {0.0f, 0.0f};
#pragma unroll
        for (int r = 0; r < 2; r++) {           // finite: the warp has at least one key that every row sees
            mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
            mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
        }
        uint32_t ph[2][4], pl[2][4];            // the 16-row operand of the two k-steps of 16 keys, high and low parts
#pragma unroll
        for (int nb = 0; nb < 4; nb++) {
            const float p0 = dm_ex2(s[nb][0] - mx[0]), p1 = dm_ex2(s[nb][1] - mx[0]);
            const float p2 = dm_ex2(s[nb][2] - mx[1]), p3 = dm_ex2(s[nb][3] - mx[1]);
            rs[0] += p0 + p1;
            rs[1] += p2 + p3;
            const __nv_bfloat162 h01 = __floats2bfloat162_rn(p0, p1), h23 = __floats2bfloat162_rn(p2, p3);
            const int kk = nb >> 1, hi = (nb & 1) * 2;
            ph[kk][hi] = *reinterpret_cast<const uint32_t*>(&h01);
            ph[kk][hi + 1] = *reinterpret_cast<const uint32_t*>(&h23);
            pl[kk][hi] = dm_pack(p0 - __bfloat162float(h01.x), p1 - __bfloat162float(h01.y));
            pl[kk][hi + 1] = dm_pack(p2 - __bfloat162float(h23.x), p3 - __bfloat162float(h23.y));
        }
#pragma unroll
        for (int r = 0; r < 2; r++) {
            rs[r] += __shfl_xor_sync(0xffffffffu, rs[r], 1);
            rs[r] += __shfl_xor_sync(0xffffffffu, rs[r], 2);
        }
        if (qd == 0) {
            *reinterpret_cast<float2*>(wml + (warp * DM_ROWS + gq) * 2) = make_float2(mx[0], rs[0]);
            *reinterpret_cast<float2*>(wml + (warp * DM_ROWS + gq + 8) * 2) = make_float2(mx[1], rs[1]);
        }

        // ---- p * v over the warp's keys, all head dimensions ------------------------------------------------
        float o[DBLK][4];
#pragma unroll
        for (int db = 0; db < DBLK; db++) { o[db][0] = o[db][1] = o[db][2] = o[db][3] = 0.0f; }
#pragma unroll
        for (int kk = 0; kk < 2; kk++) {
#pragma unroll
            for (int db = 0; db < DBLK; db += 2) {
                uint32_t b0, b1, b2, b3;
                dm_ldsm_x4_trans(b0, b1, b2, b3, sv + (warp * 32 + kk * 16 + (lane & 15)) * LD + (db + (lane >> 4)) * 8);
                dm_mma(o[db], ph[kk], b0, b1);
                dm_mma(o[db], pl[kk], b0, b1);
                dm_mma(o[db + 1], ph[kk], b2, b3);
                dm_mma(o[db + 1], pl[kk], b2, b3);
            }
        }
        __syncwarp();                           // every lane is past its reads of the warp's keys
#pragma unroll
        for (int db = 0; db < DBLK; db++) {
            const int d = db * 8 + qd * 2;
            if (gq < gt) *reinterpret_cast<float2*>(wo + gq * HD + d) = make_float2(o[db][0], o[db][1]);
            if (gq + 8 < gt) *reinterpret_cast<float2*>(wo + (gq + 8) * HD + d) = make_float2(o[db][2], o[db][3]);
        }
    } else if (lane < DM_ROWS) {
        *reinterpret_cast<float2*>(wml + (warp * DM_ROWS + lane) * 2) = make_float2(-INFINITY, 0.0f);
    }
    __syncthreads();

    // ---- the warps' parts meet: every thread takes one output element and weighs the eight parts itself, in warp
    // order (row maximum, weights exp(own maximum - row maximum), sum); the threads of a row's first column also
    // leave the row's maximum and sum
    const bool single = n_active == 1;
    for (int i = tid; i < gt * HD; i += DM_THREADS) {
        const int row = i / HD, d = i % HD;
        float2 ml[8];
#pragma unroll
        for (int w = 0; w < 8; w++) ml[w] = *reinterpret_cast<const float2*>(wml + (w * DM_ROWS + row) * 2);
        float m = ml[0].x;
#pragma unroll
        for (int w = 1; w < 8; w++) m = fmaxf(m, ml[w].x);
        float l = 0.0f, acc = 0.0f;
#pragma unroll
        for (int w = 0; w < 8; w++) {
            if (ml[w].x == -INFINITY) continue;     // a warp without a counted key left nothing
            const float e = dm_ex2(ml[w].x - m);
            l += ml[w].y * e;
            acc += reinterpret_cast<const float*>(sk + w * 32 * LD)[row * HD + d] * e;
        }
        if (single) {
            a.out[((size_t)t * nh + h0 + row) * HD + d] = __float2bfloat16_rn(acc / l);
        } else {
            a.part_o[(((size_t)zi * nh + h0 + row) * max_splits + split) * HD + d] = acc;
            if (d == 0) *reinterpret_cast<float2*>(a.part_ml + (((size_t)zi * nh + h0 + row) * max_splits + split) * 2) = make_float2(m, l);
        }
    }
    if (single) return;

    // ---- the last block of this (token, kv-head tile) combines ----------------------------------------------
    // The block's partial is written; the barrier orders it before thread 0's counting, which releases it to the
    // other blocks and acquires theirs (one instruction instead of a fence in every thread).
    __syncthreads();
    int* counter = a.counters + (size_t)zi * a.counter_tiles + it.y;
    if (tid == 0) {
        int old;
        asm volatile("atom.acq_rel.gpu.global.add.s32 %0, [%1], 1;" : "=r"(old) : "l"(counter) : "memory");
        is_last = old == n_active - 1;
        if (is_last) *counter = 0;              // ready for the next launch
    }
    __syncthreads();
    if (!is_last) return;
    // Every thread combines one output element on its own: the splits' maxima, sums and partial outputs are asked
    // for sixteen splits at a time in one trip to the second-level cache (contexts of up to 4,096 positions in one
    // trip), and folded into a running maximum, sum and output in split order (the same order whatever else is in
    // the batch).
    constexpr int TRIP = 16;
    for (int i = tid; i < gt * HD; i += DM_THREADS) {
        const int h = i / HD, d = i % HD;
        const float2* ml = reinterpret_cast<const float2*>(a.part_ml) + ((size_t)zi * nh + h0 + h) * max_splits + first_split;
        const float* po = a.part_o + (((size_t)zi * nh + h0 + h) * max_splits + first_split) * HD + d;
        float mm = -INFINITY, l = 0.0f, o = 0.0f;
        for (int j0 = 0; j0 < n_active; j0 += TRIP) {
            float2 st[TRIP];
            float pv[TRIP];
#pragma unroll
            for (int j = 0; j < TRIP; j++) {
                const bool on = j0 + j < n_active;
                st[j] = on ? __ldcg(ml + j0 + j) : make_float2(-INFINITY, 0.0f);
                pv[j] = on ? __ldcg(po + (size_t)(j0 + j) * HD) : 0.0f;
            }
            float cm = mm;
#pragma unroll
            for (int j = 0; j < TRIP; j++) cm = fmaxf(cm, st[j].x);
            const float keep = mm == -INFINITY ? 0.0f : dm_ex2(mm - cm);        // cm is finite: every split has a counted key; maxima are in base 2
            l *= keep;
            o *= keep;
#pragma unroll
            for (int j = 0; j < TRIP; j++) {
                const float e = st[j].x == -INFINITY ? 0.0f : dm_ex2(st[j].x - cm);
                l += st[j].y * e;
                o += pv[j] * e;
            }
            mm = cm;
        }
        a.out[((size_t)t * nh + h0 + h) * HD + d] = __float2bfloat16_rn(o / l);
    }
}

template <int HD>
static int launch_dm(const void* q, const void* cache, const int32_t* bt, const int32_t* token_seg, const int32_t* positions,
                     const int32_t* tok_list, void* out, float* part_o, float* part_ml, int* counters, int n_tokens, int nh, int nkv,
                     int page_size, int max_blocks, int splits, int grid_splits, int counter_tiles, float scale, int window,
                     cudaStream_t stream) {
    const int g = nh / nkv, tiles = nkv * ((g + DM_ROWS - 1) / DM_ROWS);
    int shift = -1;
    for (int b = 0; b < 30; b++) if ((1 << b) == page_size) shift = b;
    DmArgs a{(const __nv_bfloat16*)q, (const __nv_bfloat16*)cache, bt, token_seg, positions, tok_list, (__nv_bfloat16*)out, part_o,
             part_ml, counters, nh, nkv, page_size, shift, max_blocks, splits, counter_tiles, scale, window};
    // Three blocks a multiprocessor pay when there are several waves of blocks; with a single wave (a small batch)
    // two blocks and a larger first-level cache were measured faster, so the small launch asks for more shared
    // memory than it uses.
    const long long blocks = (long long)n_tokens * tiles * grid_splits;
    size_t smem = DmSmem<HD>::BYTES;
    if (blocks < 3 * 148 * 2 && smem < 100 * 1024) smem = 100 * 1024;
    auto kern = attention_decode_mma_kernel<HD>;
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
    }
    return launch_dependent(kern, dim3(grid_splits, tiles, n_tokens), dim3(DM_THREADS), smem, stream, a);
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
