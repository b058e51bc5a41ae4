// Causal attention of prompt portions over the paged cache on the fifth-generation tensor cores (bfloat16, head
// size 64): softmax(q k^T * scale) v with float32 scores, running maxima and sums (the softmax of
// engine/src/model.c:932-956, computed tile by tile).
//
// Two kernels share the decomposition, the scratch and the result; the launcher takes one or the other by the size of
// the launch (see there).  In both, one block takes a tile of up to 128 consecutive tokens of one request and one query
// head, and walks over the request's keys 64 at a time.  The first kernel:
//
//   warp 8   TMA: the query tile once; per step the keys and values of the step's pages, straight from the cache
//            (a box of one page's rows for one key-value head, 128-byte swizzle) into two three-stage rings
//   warp 9   one lane issues tcgen05.mma: S[128 x 64] = Q K^T into one of two score buffers in tensor memory (the
//            next step's scores are computed while the softmax warps work on this step's), and, once the
//            probabilities lie in shared memory, O[128 x 64] += P V (V as it lies in the cache: the N-major operand);
//            the probabilities have two buffers too, so that the softmax warps write a step's while the tensor core
//            still reads the step's before
//   warps 0-7  two threads a query row (warps w and w+4 share rows 32w .. 32w+31 and take 32 of the step's keys
//            each): read the scores from tensor memory, mask, maximum (the two meet once a step), 2^x, write the
//            probabilities as a high and a low bfloat16 part (p = hi + lo to about 2^-17, so that P V matches
//            float32 probabilities) in the swizzled K-major layout the tensor core reads
//
// O stays in tensor memory for the whole walk.  A row's reference maximum is only raised when the step's maximum
// exceeds it by more than 2^8 (then the warp scales its rows of O and the row's sum); until then the
// probabilities are taken against the older maximum and may reach 256, which float32 sums and the two bfloat16
// parts hold as well as values up to 1.  The result is normalised by the row's sum at the end.
//
// In a launch with few blocks (a portion of a few hundred tokens far into a context) a long walk is cut: a block takes at
// most AT_PART key steps of its tile (part p of a tile is steps 16p .. 16p+15 from the tile's first), so that more
// multiprocessors share the work.  A tile with one part is finished by its block as before; otherwise every part leaves its
// unnormalised output, reference maxima and sums in scratch memory, and the part that arrives last (a counter per tile
// and head, no waiting) adds them in part order and writes the result.
//
// A row's result does not depend on what else is in the batch: its keys are walked in 64s from absolute position
// 0 (or the window's first tile), parts lie at fixed steps of that walk, and every decision above is the row's own.
//
// Every wait on an mbarrier is bounded: after the launch's limit (about a second unless the host set another) the
// waiter sets *error (a word the host reads), the block stops, and its tensor memory is freed.
//
// tiles [n_tiles][4] int32: first token (flat index), rows (1..128), position of the first token, segment.
#include "tcgen05_common.cuh"

namespace vk {

constexpr int AT_BM = 128, AT_BN = 64, AT_THREADS = 320, AT_STAGES = 3;
constexpr int AT_PART = 16;          // key steps of 64 a block walks at most, where walks are cut

// Scratch of the parts: outputs [tiles][heads][parts][128][64] float32, then maxima and sums [tiles][heads][parts][128][2],
// then counters [tiles][heads] (zero before the first launch; the kernel leaves them zero).
struct AtScratch {
    float* part_o;
    float* part_ml;
    int* counters;
    int parts;                       // parts a tile can have in this launch (the grid's width is tiles * parts)
    int part_steps;                  // key steps of a part (AT_PART; an experiment may set another through VITNA_ATT_PART)
    int n_tiles;
};

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ float at_ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ uint32_t at_pack(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

// DBUF: two buffers of probabilities (132 KB of shared memory, one block a multiprocessor) instead of one (96 KB, two
// blocks): the softmax warps then write a step's probabilities while the tensor core still reads the step's before.
// Measured, that loses where two blocks can share a multiprocessor, and where they cannot the kernel with two streams
// further down is faster still: only the form with one buffer is launched.
template <int HD, bool DBUF>
__global__ void __launch_bounds__(AT_THREADS, DBUF ? 1 : 2) attention_prefill_tcgen05_kernel(
    const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_kv, const int32_t* __restrict__ block_tables,
    const int32_t* __restrict__ tiles, __nv_bfloat16* __restrict__ out, int nh, int nkv, int page_size, int max_blocks, float scale,
    int window, const WaitCtl wc, const AtScratch sc) {
    static_assert(HD == 64, "one 128-byte row per key");
    constexpr int STAGES = AT_STAGES;
    constexpr uint32_t Q_BYTES = AT_BM * HD * 2, KV_BYTES = AT_BN * HD * 2, P_BYTES = AT_BM * AT_BN * 2;
    constexpr uint32_t K_OFF = Q_BYTES, V_OFF = K_OFF + STAGES * KV_BYTES, PH_OFF = V_OFF + STAGES * KV_BYTES, PL_OFF = PH_OFF + (DBUF ? 2 : 1) * P_BYTES,
                       BAR_OFF = PL_OFF + (DBUF ? 2 : 1) * P_BYTES;
    // the probabilities of step i lie in buffer pbuf(i); its completions on p_full and pv_done have parity ppar(i)
    auto pbuf = [](int i) -> int { return DBUF ? (i & 1) : 0; };
    auto ppar = [](int i) -> uint32_t { return DBUF ? ((i >> 1) & 1) : (i & 1); };
    constexpr uint32_t TMEM_COLS = 256;              // S in columns 0..63 and 64..127 (two buffers), O in 128..191
    constexpr float RAISE = 8.0f;                    // the reference maximum follows when the step's exceeds it by 2^8
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint64_t* q_full = reinterpret_cast<uint64_t*>(smem + BAR_OFF);
    uint64_t* k_full = q_full + 1;                   // [STAGES] each: the keys' ring and the values' ring are released
    uint64_t* k_empty = k_full + STAGES;             // separately, the keys' as soon as their scores are computed
    uint64_t* v_full = k_empty + STAGES;
    uint64_t* v_empty = v_full + STAGES;
    uint64_t* s_full = v_empty + STAGES;             // [2]
    uint64_t* p_full = s_full + 2;                   // [2]: the probabilities of step i lie in buffer i & 1
    uint64_t* pv_done = p_full + 2;                  // [2]: P V of step i has read buffer i & 1 (and added into O)
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(pv_done + 2);
    __shared__ int failed, is_last;
    __shared__ float xmax[4 * AT_BM];              // the halves' maxima of a row, two steps deep; at the end their sums

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // Blocks in the order of their tiles, last tile first, all heads and parts of a tile together: later tiles of a
    // prompt walk over more keys, and a launch ends sooner when its longest blocks start first.  (Measured at 32 heads
    // and 2,048 tokens: 84 -> 62 microseconds against the order head by head.)
    const int per_tile = sc.parts * nh;
    const int tile = sc.n_tiles - 1 - blockIdx.x / per_tile, part = (blockIdx.x % per_tile) / nh;
    const int h = blockIdx.x % nh;
    const int kvh = h / (nh / nkv);
    const int tok0 = tiles[tile * 4 + 0], rows = tiles[tile * 4 + 1], pos0 = tiles[tile * 4 + 2], seg = tiles[tile * 4 + 3];
    const int last_pos = pos0 + rows - 1;
    const int lo_first = (window > 0 && pos0 - window + 1 > 0) ? pos0 - window + 1 : 0;     // lowest key any row needs
    const int kt_first = lo_first / AT_BN, kt1 = last_pos / AT_BN;      // the tile's walk: key steps kt_first .. kt1
    const int n_parts = (kt1 - kt_first) / sc.part_steps + 1;           // parts of this tile
    if (part >= n_parts) return;                                        // the whole block: nothing to do
    const int kt0 = kt_first + part * sc.part_steps;                    // this block's steps: kt0 .. kt0 + n_it - 1
    const int n_it = min(sc.part_steps, kt1 - kt0 + 1);

    if (threadIdx.x == 0) {
        failed = 0;
        mbar_init(q_full, 1);
        for (int s = 0; s < STAGES; s++) { mbar_init(&k_full[s], 1); mbar_init(&k_empty[s], 1); mbar_init(&v_full[s], 1); mbar_init(&v_empty[s], 1); }
        mbar_init(&s_full[0], 1);
        mbar_init(&s_full[1], 1);
        mbar_init(&p_full[0], 2 * AT_BM);
        mbar_init(&p_full[1], 2 * AT_BM);
        mbar_init(&pv_done[0], 1);
        mbar_init(&pv_done[1], 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 9) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_s = *tmem_slot, tmem_o = tmem_s + 2 * AT_BN;

    if (warp == 8) {
        // ---- producer ------------------------------------------------------------------------------------
        if (lane == 0) {
            mbar_expect_tx(q_full, Q_BYTES);
            tma_load_2d(smem, &map_q, h * HD, tok0, q_full);      // rows beyond the batch read as zero
        }
        const int32_t* bt = block_tables + (size_t)seg * max_blocks;
        const int box_rows = page_size < AT_BN ? page_size : AT_BN, boxes = AT_BN / box_rows;
        // Lane b takes box b of a step.  The pages come from the block table 32 at a time (lane l the l-th page from the
        // batch's first: the pages of 32 * page_size / 64 steps), a batch ahead of their use, and are handed round by
        // shuffle: a trip to the block table in every step paced the whole walk (a step took as long as the trip).
        const int batch_steps = 32 * page_size / AT_BN, last_page = last_pos / page_size;      // >= 4: pages hold at least 8 keys
        auto load_batch = [&](int i0) -> int {
            const int p0 = ((kt0 + i0) * AT_BN) / page_size;
            return (i0 < n_it && p0 + lane <= last_page) ? bt[p0 + lane] : 0;
        };
        int pages_now = load_batch(0), pages_next = load_batch(batch_steps), batch_first = 0;
        for (int i = 0; i < n_it; i++) {
            const int s = i % STAGES, key0 = (kt0 + i) * AT_BN;
            if (i - batch_first == batch_steps) {
                batch_first = i;
                pages_now = pages_next;
                pages_next = load_batch(i + batch_steps);
            }
            const int page = __shfl_sync(0xffffffffu, pages_now, ((key0 + lane * box_rows) / page_size - ((kt0 + batch_first) * AT_BN) / page_size) & 31);
            // boxes that hold a key some row needs; the rows of the others are never counted (p = 0) and the
            // values' rows beyond the last position are zeroed by the softmax warps
            int nb = (last_pos - key0) / box_rows + 1;
            nb = nb < boxes ? nb : boxes;
            const int off = (key0 + lane * box_rows) % page_size;
            const uint32_t dst = s * KV_BYTES + lane * box_rows * (HD * 2);
            if (i >= STAGES) {
                const bool ok = mbar_wait(&k_empty[s], ((i / STAGES) - 1) & 1, wc.cycles);
                if (!__all_sync(0xffffffffu, ok)) { if (lane == 0) give_up(wc.error, &failed, 11); break; }
            }
            if (i != wc.skip_stage) {          // (a step named by wc.skip_stage gets no keys: a test of the give-up path)
                if (lane == 0) mbar_expect_tx(&k_full[s], (uint32_t)nb * box_rows * HD * 2);
                __syncwarp();
                if (lane < nb) tma_load_2d(smem + K_OFF + dst, &map_kv, 0, (page * 2 * nkv + kvh) * page_size + off, &k_full[s]);
            }
            if (i >= STAGES) {
                const bool ok = mbar_wait(&v_empty[s], ((i / STAGES) - 1) & 1, wc.cycles);
                if (!__all_sync(0xffffffffu, ok)) { if (lane == 0) give_up(wc.error, &failed, 19); break; }
            }
            if (lane == 0) mbar_expect_tx(&v_full[s], (uint32_t)nb * box_rows * HD * 2);
            __syncwarp();
            if (lane < nb) tma_load_2d(smem + V_OFF + dst, &map_kv, 0, ((page * 2 + 1) * nkv + kvh) * page_size + off, &v_full[s]);
        }
    } else if (warp == 9) {
        // ---- tensor core ---------------------------------------------------------------------------------
        if (lane == 0) {
            const uint32_t idesc_qk = umma_idesc_bf16(AT_BM, AT_BN);
            const uint32_t idesc_pv = umma_idesc_bf16(AT_BM, HD) | (1u << 16);        // B (the values) is N-major
            // the low words of the operands' descriptors (see umma_bf16_lo): stepped by bytes / 16
            const uint32_t q_lo = umma_desc_lo(smem_u32(smem)), k_lo0 = umma_desc_lo(smem_u32(smem + K_OFF)), v_lo0 = umma_desc_lo(smem_u32(smem + V_OFF));
            const uint32_t ph_lo0 = umma_desc_lo(smem_u32(smem + PH_OFF)), pl_lo0 = umma_desc_lo(smem_u32(smem + PL_OFF));
            auto scores = [&](int i) -> bool {        // S[i & 1] = Q K_i^T
                const int s = i % STAGES;
                if (!mbar_wait(&k_full[s], (i / STAGES) & 1, wc.cycles)) { give_up(wc.error, &failed, 13); return false; }
                tc_fence_after();
                const uint32_t k_lo = k_lo0 + s * (KV_BYTES >> 4), s_addr = tmem_s + (i & 1) * AT_BN;
#pragma unroll
                for (int k = 0; k < HD / 16; k++) umma_bf16_lo(s_addr, q_lo + 2 * k, k_lo + 2 * k, idesc_qk, k != 0);
                umma_commit(&s_full[i & 1]);
                umma_commit(&k_empty[s]);               // the keys' stage is free once these instructions have read it
                return true;
            };
            bool ok = mbar_wait(q_full, 0, wc.cycles);
            if (!ok) give_up(wc.error, &failed, 12);
            ok = ok && scores(0);
            for (int i = 0; i < n_it && ok; i++) {
                // the next step's scores go into the other buffer while the softmax warps work on this step's
                if (i + 1 < n_it && !scores(i + 1)) break;
                if (!mbar_wait(&v_full[i % STAGES], (i / STAGES) & 1, wc.cycles)) { give_up(wc.error, &failed, 20); break; }
                if (!mbar_wait(&p_full[pbuf(i)], ppar(i), wc.cycles)) { give_up(wc.error, &failed, 14); break; }
                const uint32_t pb = (uint32_t)pbuf(i) * (P_BYTES >> 4);
                tc_fence_after();
                const uint32_t v_lo = v_lo0 + (i % STAGES) * (KV_BYTES >> 4), ph_lo = ph_lo0 + pb, pl_lo = pl_lo0 + pb;
                // 16 keys an instruction: two groups of eight 128-byte rows of the values
#pragma unroll
                for (int k = 0; k < AT_BN / 16; k++) umma_bf16_lo(tmem_o, ph_lo + 2 * k, v_lo + k * (2048 >> 4), idesc_pv, (i | k) != 0);
#pragma unroll
                for (int k = 0; k < AT_BN / 16; k++) umma_bf16_lo(tmem_o, pl_lo + 2 * k, v_lo + k * (2048 >> 4), idesc_pv, 1);
                umma_commit(&v_empty[i % STAGES]);
                umma_commit(&pv_done[pbuf(i)]);
            }
        }
    } else {
        // ---- softmax: two threads a query row, 32 of the step's 64 keys each -----------------------------------
        const int half = warp >> 2;                  // which 32 keys of a step, and which 32 columns of O
        const int r = (warp & 3) * 32 + lane;
        const bool valid = r < rows;
        const int my_pos = pos0 + r;
        const int my_lo = (window > 0 && my_pos - window + 1 > 0) ? my_pos - window + 1 : 0;
        const float scale_log2 = scale * 1.4426950408889634f;
        const uint32_t lane_off = (uint32_t)((warp & 3) * 32) << 16;
        const uint32_t bar_id = 1 + (warp & 3);      // the two warps of a row quarter meet on this barrier
        uint8_t* ph_row = smem + PH_OFF + r * 128;
        uint8_t* pl_row = smem + PL_OFF + r * 128;
        float m = -INFINITY, l = 0.0f;              // the row's reference maximum (log2 units) and this half's sum against it
        // A failed wait clears `ok`; the thread then only keeps meeting its partner and arriving, so that nobody
        // waits for it without a limit.
        bool ok = true;
        for (int i = 0; i < n_it; i++) {
            const int key0 = (kt0 + i) * AT_BN + half * 32;
            uint32_t sr[32];
            float mx = -INFINITY;
            if (ok && !__all_sync(0xffffffffu, mbar_wait(&s_full[i & 1], (i >> 1) & 1, wc.cycles))) { if (lane == 0) give_up(wc.error, &failed, 15); ok = false; }
            if (ok) {
                tc_fence_after();
                tmem_ld32(tmem_s + (i & 1) * AT_BN + half * 32 + lane_off, sr);
                tmem_loaded(sr);
                // raw scores: the maximum commutes with the (positive) scale; masked keys become -inf only on tiles
                // that touch the diagonal, the window's edge or rows beyond the tile's own
                if (!valid || key0 + 31 > my_pos || key0 < my_lo) {
#pragma unroll
                    for (int j = 0; j < 32; j++) {
                        const int kk = key0 + j;
                        if (!(valid && kk <= my_pos && kk >= my_lo)) sr[j] = 0xff800000u;
                    }
                }
#pragma unroll
                for (int j = 0; j < 32; j++) mx = fmaxf(mx, __uint_as_float(sr[j]));
                mx *= scale_log2;
            }
            xmax[((i & 1) * 2 + half) * AT_BM + r] = mx;
            asm volatile("bar.sync %0, 64;" ::"r"(bar_id) : "memory");
            mx = fmaxf(mx, xmax[((i & 1) * 2 + (half ^ 1)) * AT_BM + r]);
            if (i == 0) {
                m = mx;                             // O is written, not added to, by the first step
            } else if (ok) {
                const bool raise = mx > m + RAISE;  // also the first counted key after none (m = -inf)
                if (__any_sync(0xffffffffu, raise)) {
                    // scale this warp's part of O (and the sums) to the new maxima; every earlier P V must have landed
                    if (!__all_sync(0xffffffffu, mbar_wait(&pv_done[pbuf(i - 1)], ppar(i - 1), wc.cycles))) { if (lane == 0) give_up(wc.error, &failed, 16); ok = false; }
                    if (ok) {
                        tc_fence_after();
                        const float alpha = raise ? at_ex2(m - mx) : 1.0f;
                        uint32_t orr[32];
                        tmem_ld32(tmem_o + lane_off + half * 32, orr);
                        tmem_loaded(orr);
#pragma unroll
                        for (int j = 0; j < 32; j++) orr[j] = __float_as_uint(__uint_as_float(orr[j]) * alpha);
                        tmem_st32(tmem_o + lane_off + half * 32, orr);
                        tmem_wait_st();
                        l *= alpha;
                        if (raise) m = mx;
                    }
                }
            }
            const float m_use = m == -INFINITY ? 0.0f : m;
            // the probabilities of this step replace those of the step that had the buffer last, once its P V has read them
            // (with two buffers that is the step before last, and the step before this one may still be under way)
            const int had = DBUF ? i - 2 : i - 1;
            if (ok && had >= 0) {
                if (!__all_sync(0xffffffffu, mbar_wait(&pv_done[pbuf(had)], ppar(had), wc.cycles))) { if (lane == 0) give_up(wc.error, &failed, 17); ok = false; }
            }
            if (ok) {
                float sum = 0.0f;
#pragma unroll
                for (int j8 = 0; j8 < 32; j8 += 8) {
                    uint32_t hi[4], lo[4];
#pragma unroll
                    for (int j = 0; j < 8; j += 2) {
                        const float p0 = at_ex2(fmaf(__uint_as_float(sr[j8 + j]), scale_log2, -m_use));
                        const float p1 = at_ex2(fmaf(__uint_as_float(sr[j8 + j + 1]), scale_log2, -m_use));
                        sum += p0 + p1;
                        const __nv_bfloat162 hv = __floats2bfloat162_rn(p0, p1);
                        hi[j / 2] = *reinterpret_cast<const uint32_t*>(&hv);
                        lo[j / 2] = at_pack(p0 - __bfloat162float(hv.x), p1 - __bfloat162float(hv.y));
                    }
                    const int chunk = (half * 4 + (j8 >> 3)) ^ (r & 7);      // 128-byte swizzle: 16-byte piece index xor row mod 8
                    *reinterpret_cast<uint4*>(ph_row + pbuf(i) * P_BYTES + chunk * 16) = make_uint4(hi[0], hi[1], hi[2], hi[3]);
                    *reinterpret_cast<uint4*>(pl_row + pbuf(i) * P_BYTES + chunk * 16) = make_uint4(lo[0], lo[1], lo[2], lo[3]);
                }
                l += sum;
                // the values' rows beyond the last position (pages not loaded, slots not yet written): never counted,
                // but 0 * garbage must not be NaN
                if (kt0 + i == kt1 && (last_pos & (AT_BN - 1)) != AT_BN - 1 &&
                    __all_sync(0xffffffffu, mbar_wait(&v_full[i % STAGES], (i / STAGES) & 1, wc.cycles))) {      // the values have landed
                    const int z0 = (last_pos & (AT_BN - 1)) + 1;
                    uint8_t* vs = smem + V_OFF + (i % STAGES) * KV_BYTES;
                    for (int idx = half * AT_BM + r; idx < (AT_BN - z0) * 8; idx += 2 * AT_BM)
                        *reinterpret_cast<uint4*>(vs + (z0 + idx / 8) * 128 + (idx & 7) * 16) = make_uint4(0, 0, 0, 0);
                }
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // P (and the zeros) are for the tensor core
                tc_fence_before();
            }
            mbar_arrive(&p_full[pbuf(i)]);
        }
        // the row's sum is the two halves' (both against the same maximum)
        xmax[half * AT_BM + r] = l;
        asm volatile("bar.sync %0, 64;" ::"r"(bar_id) : "memory");
        l += xmax[(half ^ 1) * AT_BM + r];
        if (ok && !__all_sync(0xffffffffu, mbar_wait(&pv_done[pbuf(n_it - 1)], ppar(n_it - 1), wc.cycles))) { if (lane == 0) give_up(wc.error, &failed, 18); ok = false; }
        uint32_t orr[32];
        if (ok) {
            tc_fence_after();
            tmem_ld32(tmem_o + lane_off + half * 32, orr);
            tmem_loaded(orr);
        }
        if (n_parts == 1) {
            if (ok && valid) {
                const float inv = 1.0f / l;
                __nv_bfloat16* dst = out + ((size_t)(tok0 + r) * nh + h) * HD + half * 32;
#pragma unroll
                for (int d = 0; d < 32; d += 8) {
                    uint4 v;
                    v.x = at_pack(__uint_as_float(orr[d]) * inv, __uint_as_float(orr[d + 1]) * inv);
                    v.y = at_pack(__uint_as_float(orr[d + 2]) * inv, __uint_as_float(orr[d + 3]) * inv);
                    v.z = at_pack(__uint_as_float(orr[d + 4]) * inv, __uint_as_float(orr[d + 5]) * inv);
                    v.w = at_pack(__uint_as_float(orr[d + 6]) * inv, __uint_as_float(orr[d + 7]) * inv);
                    *reinterpret_cast<uint4*>(dst + d) = v;
                }
            }
        } else {
            // this part's unnormalised output, reference maximum and sum; a row without a counted key in this part
            // (its keys all lie in earlier parts) leaves maximum -inf and nothing else
            const size_t slot = ((size_t)tile * nh + h) * sc.parts + part;
            float* po = sc.part_o + (slot * AT_BM + r) * HD + half * 32;
            if (ok && valid) {
#pragma unroll
                for (int d = 0; d < 32; d += 4)
                    *reinterpret_cast<float4*>(po + d) = make_float4(__uint_as_float(orr[d]), __uint_as_float(orr[d + 1]), __uint_as_float(orr[d + 2]),
                                                                     __uint_as_float(orr[d + 3]));
                if (half == 0) *reinterpret_cast<float2*>(sc.part_ml + (slot * AT_BM + r) * 2) = make_float2(m, l);
            }
            // The 256 softmax threads meet; thread 0's counting releases the block's partial and acquires the others'.
            // (A block whose wait ran out counts too, so that the counter returns to zero; the error word says that
            // the result is not valid.)
            asm volatile("bar.sync 5, 256;" ::: "memory");
            if (threadIdx.x == 0) {
                int* counter = sc.counters + (size_t)tile * nh + h;
                int old;
                asm volatile("atom.acq_rel.gpu.global.add.s32 %0, [%1], 1;" : "=r"(old) : "l"(counter) : "memory");
                is_last = old == n_parts - 1;
                if (is_last) *counter = 0;          // ready for the next launch
            }
            asm volatile("bar.sync 5, 256;" ::: "memory");
            if (is_last && valid) {
                // parts in part order: running maximum, weights 2^(part's maximum - maximum), sum, output
                const size_t first = ((size_t)tile * nh + h) * sc.parts;
                float mm = -INFINITY, ll = 0.0f, acc[32];
#pragma unroll
                for (int d = 0; d < 32; d++) acc[d] = 0.0f;
                for (int j = 0; j < n_parts; j++) {
                    const float2 ml = __ldcg(reinterpret_cast<const float2*>(sc.part_ml + ((first + j) * AT_BM + r) * 2));
                    if (ml.x == -INFINITY) continue;
                    const float cm = fmaxf(mm, ml.x);
                    const float keep = mm == -INFINITY ? 0.0f : at_ex2(mm - cm), w = at_ex2(ml.x - cm);
                    const float4* src = reinterpret_cast<const float4*>(sc.part_o + ((first + j) * AT_BM + r) * HD + half * 32);
                    ll = ll * keep + ml.y * w;
#pragma unroll
                    for (int d = 0; d < 32; d += 4) {
                        const float4 v = __ldcg(src + d / 4);
                        acc[d] = acc[d] * keep + v.x * w; acc[d + 1] = acc[d + 1] * keep + v.y * w;
                        acc[d + 2] = acc[d + 2] * keep + v.z * w; acc[d + 3] = acc[d + 3] * keep + v.w * w;
                    }
                    mm = cm;
                }
                const float inv = 1.0f / ll;
                __nv_bfloat16* dst = out + ((size_t)(tok0 + r) * nh + h) * HD + half * 32;
#pragma unroll
                for (int d = 0; d < 32; d += 8) {
                    uint4 v;
                    v.x = at_pack(acc[d] * inv, acc[d + 1] * inv);
                    v.y = at_pack(acc[d + 2] * inv, acc[d + 3] * inv);
                    v.z = at_pack(acc[d + 4] * inv, acc[d + 5] * inv);
                    v.w = at_pack(acc[d + 6] * inv, acc[d + 7] * inv);
                    *reinterpret_cast<uint4*>(dst + d) = v;
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 9) {
        if (failed) __nanosleep(200000);      // after a failed wait: let copies in flight land
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_s), "r"(TMEM_COLS) : "memory");
    }
}

// ---------------------------------------------------------------------------------------------------------------
// The form with two independent streams of key steps, for launches that give a multiprocessor one or two blocks.
//
// Above, the two threads of a query row meet once a step, a step's softmax is one long chain of dependent latencies
// (scores out of tensor memory, maximum, meeting, 2^x, the probabilities into shared memory, the fence), and one
// warp makes all the copies and one lane issues all the products: with a single block on a multiprocessor a step of
// 64 keys takes 1,850 cycles, of which the tensor core works 600.  Here
//
//   * a thread owns a whole query row, and the eight softmax warps are two groups that never meet during the walk:
//     group g takes the steps i with i mod 2 = g and has its own score buffer, probability buffer, output accumulator
//     in tensor memory, reference maxima and sums, exactly as if the even and the odd key steps were two parts of the
//     walk.  While one group is in its chain the other is in its own, about half a step apart.  At the end group 1
//     hands its rows to group 0 through shared memory, and the two streams are added like two parts
//     (weights 2^(own maximum - common maximum));
//   * the scores run two steps ahead: a group tells (s_free) when it has a step's scores in registers, and its buffer
//     is written again at once;
//   * four warps serve them: one copies the keys, one the values (a copy of a page's 16 rows costs its issuer about
//     65 cycles, eight of them a step paced the walk), one lane issues the scores and one lane of another warp P V.
//
// Measured with a cycle counter in every role (9 heads, 2,048 tokens): a step takes 1,400 cycles, a group's chain
// 1,850 of computing for its step of two; what is left is the issue slots that the four serving warps and the
// eight softmax warps share.
// ---------------------------------------------------------------------------------------------------------------
constexpr int AS_STAGES = 6, AS_THREADS = 384;      // warps 0-7 softmax, 8 copies the keys, 9 issues the scores, 10 issues P V, 11 copies the values

template <int HD>
__global__ void __launch_bounds__(AS_THREADS, 1) attention_prefill_streams_kernel(
    const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_kv, const int32_t* __restrict__ block_tables,
    const int32_t* __restrict__ tiles, __nv_bfloat16* __restrict__ out, int nh, int nkv, int page_size, int max_blocks, float scale,
    int window, const WaitCtl wc, const AtScratch sc) {
    static_assert(HD == 64, "one 128-byte row per key");
    constexpr int STAGES = AS_STAGES;
    constexpr uint32_t Q_BYTES = AT_BM * HD * 2, KV_BYTES = AT_BN * HD * 2, P_BYTES = AT_BM * AT_BN * 2;
    constexpr uint32_t K_OFF = Q_BYTES, V_OFF = K_OFF + STAGES * KV_BYTES, PH_OFF = V_OFF + STAGES * KV_BYTES, PL_OFF = PH_OFF + 2 * P_BYTES,
                       BAR_OFF = PL_OFF + 2 * P_BYTES;
    constexpr uint32_t TMEM_COLS = 256;              // S of the two groups in columns 0..63 and 64..127, their O in 128..191 and 192..255
    constexpr float RAISE = 8.0f;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint64_t* q_full = reinterpret_cast<uint64_t*>(smem + BAR_OFF);
    uint64_t* k_full = q_full + 1;
    uint64_t* k_empty = k_full + STAGES;
    uint64_t* v_full = k_empty + STAGES;
    uint64_t* v_empty = v_full + STAGES;
    uint64_t* s_full = v_empty + STAGES;             // [2]: group g's scores lie in its buffer
    uint64_t* s_free = s_full + 2;                   // [2]: group g has them in registers
    uint64_t* p_full = s_free + 2;                   // [2]: group g's probabilities lie in its buffer
    uint64_t* pv_done = p_full + 2;                  // [2]: P V of group g's step has read them (and added into its O)
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(pv_done + 2);
    __shared__ int failed, is_last;
    __shared__ float2 ml1[AT_BM];                    // group 1's maxima and sums, for the end

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int per_tile = sc.parts * nh;
    const int tile = sc.n_tiles - 1 - blockIdx.x / per_tile, part = (blockIdx.x % per_tile) / nh;
    const int h = blockIdx.x % nh;
    const int kvh = h / (nh / nkv);
    const int tok0 = tiles[tile * 4 + 0], rows = tiles[tile * 4 + 1], pos0 = tiles[tile * 4 + 2], seg = tiles[tile * 4 + 3];
    const int last_pos = pos0 + rows - 1;
    const int lo_first = (window > 0 && pos0 - window + 1 > 0) ? pos0 - window + 1 : 0;
    const int kt_first = lo_first / AT_BN, kt1 = last_pos / AT_BN;
    const int n_parts = (kt1 - kt_first) / sc.part_steps + 1;
    if (part >= n_parts) return;
    const int kt0 = kt_first + part * sc.part_steps;
    const int n_it = min(sc.part_steps, kt1 - kt0 + 1);

    if (threadIdx.x == 0) {
        failed = 0;
        mbar_init(q_full, 1);
        for (int s = 0; s < STAGES; s++) { mbar_init(&k_full[s], 1); mbar_init(&k_empty[s], 1); mbar_init(&v_full[s], 1); mbar_init(&v_empty[s], 1); }
        for (int g = 0; g < 2; g++) {
            mbar_init(&s_full[g], 1);
            mbar_init(&s_free[g], 4);                // one arrival a warp of the group
            mbar_init(&p_full[g], AT_BM);
            mbar_init(&pv_done[g], 1);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 9) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_s = *tmem_slot, tmem_o = tmem_s + 2 * AT_BN;

    if (warp == 8 || warp == 11) {
        // ---- the copies: warp 8 the query tile and the keys, warp 11 the values, each into its ring of six stages --------
        // (one warp for both was what paced the walk: eight copies a step with pages of 16, about 65 cycles each to
        // issue, beside its waits)
        const bool values = warp == 11;
        if (!values && lane == 0) {
            mbar_expect_tx(q_full, Q_BYTES);
            tma_load_2d(smem, &map_q, h * HD, tok0, q_full);
        }
        const int32_t* bt = block_tables + (size_t)seg * max_blocks;
        const int box_rows = page_size < AT_BN ? page_size : AT_BN, boxes = AT_BN / box_rows;
        uint64_t* full = values ? v_full : k_full;
        uint64_t* empty = values ? v_empty : k_empty;
        uint8_t* ring = smem + (values ? V_OFF : K_OFF);
        const int which = values ? 1 : 0;
        // Lane b takes box b of a step.  The pages come from the block table 32 at a time (lane l the l-th page from the
        // batch's first: the pages of 32 * page_size / 64 steps), a batch ahead of their use, and are handed round by
        // shuffle: a trip to the block table in every step would pace the walk.
        const int batch_steps = 32 * page_size / AT_BN, last_page = last_pos / page_size;      // >= 4: pages hold at least 8 keys
        auto load_batch = [&](int i0) -> int {
            const int p0 = ((kt0 + i0) * AT_BN) / page_size;
            return (i0 < n_it && p0 + lane <= last_page) ? bt[p0 + lane] : 0;
        };
        int pages_now = load_batch(0), pages_next = load_batch(batch_steps), batch_first = 0, batch_page0 = (kt0 * AT_BN) / page_size;
        const int lane_key = lane * box_rows;
        for (int i = 0; i < n_it; i++) {
            const int s = i % STAGES, key0 = (kt0 + i) * AT_BN;
            if (i - batch_first == batch_steps) {
                batch_first = i;
                batch_page0 = key0 / page_size;
                pages_now = pages_next;
                pages_next = load_batch(i + batch_steps);
            }
            const int my_page_index = (key0 + lane_key) / page_size;
            const int page = __shfl_sync(0xffffffffu, pages_now, (my_page_index - batch_page0) & 31);
            // boxes that hold a key some row needs; the rows of the others are never counted (p = 0) and the
            // values' rows beyond the last position are zeroed by the softmax warps
            int nb = (last_pos - key0) / box_rows + 1;
            nb = nb < boxes ? nb : boxes;
            const int off = key0 + lane_key - my_page_index * page_size;
            if (i >= STAGES) {
                const bool ok = mbar_wait(&empty[s], ((i / STAGES) - 1) & 1, wc.cycles);
                if (!__all_sync(0xffffffffu, ok)) { if (lane == 0) give_up(wc.error, &failed, values ? 19 : 11); break; }
            }
            if (values || i != wc.skip_stage) {     // (a step named by wc.skip_stage gets no keys: a test of the give-up path)
                if (lane == 0) mbar_expect_tx(&full[s], (uint32_t)nb * box_rows * HD * 2);
                __syncwarp();
                if (lane < nb)
                    tma_load_2d(ring + s * KV_BYTES + lane_key * (HD * 2), &map_kv, 0, ((page * 2 + which) * nkv + kvh) * page_size + off, &full[s]);
            }
        }
    } else if (warp == 9) {
        // ---- tensor core: the scores, two steps ahead -----------------------------------------------------------
        if (lane == 0) {
            const uint32_t idesc_qk = umma_idesc_bf16(AT_BM, AT_BN);
            const uint32_t q_lo = umma_desc_lo(smem_u32(smem)), k_lo0 = umma_desc_lo(smem_u32(smem + K_OFF));
            auto scores = [&](int i) -> bool {
                const int s = i % STAGES;
                if (!mbar_wait(&k_full[s], (i / STAGES) & 1, wc.cycles)) { give_up(wc.error, &failed, 13); return false; }
                tc_fence_after();
                const uint32_t k_lo = k_lo0 + s * (KV_BYTES >> 4), s_addr = tmem_s + (i & 1) * AT_BN;
#pragma unroll
                for (int k = 0; k < HD / 16; k++) umma_bf16_lo(s_addr, q_lo + 2 * k, k_lo + 2 * k, idesc_qk, k != 0);
                umma_commit(&s_full[i & 1]);
                umma_commit(&k_empty[s]);
                return true;
            };
            bool ok = mbar_wait(q_full, 0, wc.cycles);
            if (!ok) give_up(wc.error, &failed, 12);
            ok = ok && scores(0);
            if (n_it > 1) ok = ok && scores(1);
            for (int i = 0; i + 2 < n_it && ok; i++) {
                // the group has this step's scores in registers: its buffer takes the scores of its next step
                if (!mbar_wait(&s_free[i & 1], (uint32_t)(i >> 1) & 1, wc.cycles)) { give_up(wc.error, &failed, 21); break; }
                tc_fence_after();
                if (!scores(i + 2)) break;
            }
        }
    } else if (warp == 10) {
        // ---- tensor core, the other issuer: P V as the probabilities arrive ---------------------------------------
        if (lane == 0) {
            const uint32_t idesc_pv = umma_idesc_bf16(AT_BM, HD) | (1u << 16);
            const uint32_t ph_lo0 = umma_desc_lo(smem_u32(smem + PH_OFF)), pl_lo0 = umma_desc_lo(smem_u32(smem + PL_OFF));
            const uint32_t v_lo0 = umma_desc_lo(smem_u32(smem + V_OFF));
            for (int i = 0; i < n_it; i++) {
                const int g = i & 1;
                const uint32_t par = (uint32_t)(i >> 1) & 1;
                if (!mbar_wait(&v_full[i % STAGES], (i / STAGES) & 1, wc.cycles)) { give_up(wc.error, &failed, 20); break; }
                if (!mbar_wait(&p_full[g], par, wc.cycles)) { give_up(wc.error, &failed, 14); break; }
                tc_fence_after();
                const uint32_t pb = (uint32_t)g * (P_BYTES >> 4), o_addr = tmem_o + g * HD;
                const uint32_t v_lo = v_lo0 + (i % STAGES) * (KV_BYTES >> 4), ph_lo = ph_lo0 + pb, pl_lo = pl_lo0 + pb;
#pragma unroll
                for (int k = 0; k < AT_BN / 16; k++) umma_bf16_lo(o_addr, ph_lo + 2 * k, v_lo + k * (2048 >> 4), idesc_pv, (i >= 2) || k != 0);
#pragma unroll
                for (int k = 0; k < AT_BN / 16; k++) umma_bf16_lo(o_addr, pl_lo + 2 * k, v_lo + k * (2048 >> 4), idesc_pv, 1);
                umma_commit(&v_empty[i % STAGES]);
                umma_commit(&pv_done[g]);
            }
        }
    } else {
        // ---- softmax: a thread a query row; group g = warp / 4 takes the steps i with i mod 2 = g ----------------
        const int g = warp >> 2;
        const int r = (warp & 3) * 32 + lane;
        const bool valid = r < rows;
        const int my_pos = pos0 + r;
        const int my_lo = (window > 0 && my_pos - window + 1 > 0) ? my_pos - window + 1 : 0;
        const float scale_log2 = scale * 1.4426950408889634f;
        const uint32_t lane_off = (uint32_t)((warp & 3) * 32) << 16;
        const uint32_t my_s = tmem_s + g * AT_BN + lane_off, my_o = tmem_o + g * HD + lane_off;
        uint8_t* ph_row = smem + PH_OFF + g * P_BYTES + r * 128;
        uint8_t* pl_row = smem + PL_OFF + g * P_BYTES + r * 128;
        float m = -INFINITY, l = 0.0f;              // the row's reference maximum (log2 units) and sum in this group's stream
        bool ok = true;
        int steps = 0;                              // steps this group has taken
        for (int i = g; i < n_it; i += 2, steps++) {
            const uint32_t par = (uint32_t)steps & 1;
            const int key0 = (kt0 + i) * AT_BN;
            uint32_t sr[64];
            if (ok && !__all_sync(0xffffffffu, mbar_wait(&s_full[g], par, wc.cycles))) { if (lane == 0) give_up(wc.error, &failed, 15); ok = false; }
            float mx = -INFINITY;
            if (ok) {
                tc_fence_after();
                tmem_ld32_nowait(my_s, sr);
                tmem_ld32_nowait(my_s + 32, sr + 32);
                tmem_wait_ld();
                tmem_loaded(sr);
                tmem_loaded(sr + 32);
            }
            // the scores are in registers (or the walk has failed): the buffer may take the group's next step
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&s_free[g]);
            if (ok) {
                if (!valid || key0 + AT_BN - 1 > my_pos || key0 < my_lo) {
#pragma unroll
                    for (int j = 0; j < 64; j++) {
                        const int kk = key0 + j;
                        if (!(valid && kk <= my_pos && kk >= my_lo)) sr[j] = 0xff800000u;
                    }
                }
                float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
                for (int j = 0; j < 64; j += 4) {
                    mx4[0] = fmaxf(mx4[0], __uint_as_float(sr[j]));
                    mx4[1] = fmaxf(mx4[1], __uint_as_float(sr[j + 1]));
                    mx4[2] = fmaxf(mx4[2], __uint_as_float(sr[j + 2]));
                    mx4[3] = fmaxf(mx4[3], __uint_as_float(sr[j + 3]));
                }
                mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])) * scale_log2;
            }
            // the group's last step has read this buffer of probabilities and added into O: both may change now
            if (ok && steps > 0) {
                if (!__all_sync(0xffffffffu, mbar_wait(&pv_done[g], par ^ 1, wc.cycles))) { if (lane == 0) give_up(wc.error, &failed, 17); ok = false; }
            }
            if (steps == 0) {
                m = mx;                             // O is written, not added to, by the group's first step
            } else if (ok) {
                const bool raise = mx > m + RAISE;  // also the first counted key after none (m = -inf)
                if (__any_sync(0xffffffffu, raise)) {
                    tc_fence_after();
                    const float alpha = raise ? at_ex2(m - mx) : 1.0f;
#pragma unroll
                    for (int c = 0; c < HD; c += 32) {
                        uint32_t orr[32];
                        tmem_ld32(my_o + c, orr);
                        tmem_loaded(orr);
#pragma unroll
                        for (int j = 0; j < 32; j++) orr[j] = __float_as_uint(__uint_as_float(orr[j]) * alpha);
                        tmem_st32(my_o + c, orr);
                    }
                    tmem_wait_st();
                    l *= alpha;
                    if (raise) m = mx;
                }
            }
            const float m_use = m == -INFINITY ? 0.0f : m;
            if (ok) {
                float sum0 = 0.0f, sum1 = 0.0f;
#pragma unroll
                for (int j8 = 0; j8 < 64; j8 += 8) {
                    uint32_t hi[4], lo[4];
#pragma unroll
                    for (int j = 0; j < 8; j += 2) {
                        const float p0 = at_ex2(fmaf(__uint_as_float(sr[j8 + j]), scale_log2, -m_use));
                        const float p1 = at_ex2(fmaf(__uint_as_float(sr[j8 + j + 1]), scale_log2, -m_use));
                        sum0 += p0;
                        sum1 += p1;
                        const __nv_bfloat162 hv = __floats2bfloat162_rn(p0, p1);
                        hi[j / 2] = *reinterpret_cast<const uint32_t*>(&hv);
                        lo[j / 2] = at_pack(p0 - __bfloat162float(hv.x), p1 - __bfloat162float(hv.y));
                    }
                    const int chunk = (j8 >> 3) ^ (r & 7);      // 128-byte swizzle: 16-byte piece index xor row mod 8
                    *reinterpret_cast<uint4*>(ph_row + chunk * 16) = make_uint4(hi[0], hi[1], hi[2], hi[3]);
                    *reinterpret_cast<uint4*>(pl_row + chunk * 16) = make_uint4(lo[0], lo[1], lo[2], lo[3]);
                }
                l += sum0 + sum1;
                // the values' rows beyond the last position: never counted, but 0 * garbage must not be NaN
                if (kt0 + i == kt1 && (last_pos & (AT_BN - 1)) != AT_BN - 1 &&
                    __all_sync(0xffffffffu, mbar_wait(&v_full[i % STAGES], (i / STAGES) & 1, wc.cycles))) {
                    const int z0 = (last_pos & (AT_BN - 1)) + 1;
                    uint8_t* vs = smem + V_OFF + (i % STAGES) * KV_BYTES;
                    for (int idx = r; idx < (AT_BN - z0) * 8; idx += AT_BM)
                        *reinterpret_cast<uint4*>(vs + (z0 + idx / 8) * 128 + (idx & 7) * 16) = make_uint4(0, 0, 0, 0);
                }
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                tc_fence_before();
            }
            mbar_arrive(&p_full[g]);
        }
        // ---- the end: the group's last P V has landed; group 1 hands its stream to group 0 ------------------------
        if (ok && steps > 0 && !__all_sync(0xffffffffu, mbar_wait(&pv_done[g], (uint32_t)(steps - 1) & 1, wc.cycles))) {
            if (lane == 0) give_up(wc.error, &failed, 18);
            ok = false;
        }
        float* xo = reinterpret_cast<float*>(smem + PH_OFF);        // [128][64] float32 over the probabilities' buffers, pieces of 16 bytes xor row
        if (g == 1) {
            // the rows go where the probabilities lay: group 0's last P V (the walk's last step, if their number is odd)
            // must have read them too
            if (ok && (n_it & 1) && !__all_sync(0xffffffffu, mbar_wait(&pv_done[0], (uint32_t)((n_it + 1) / 2 - 1) & 1, wc.cycles))) {
                if (lane == 0) give_up(wc.error, &failed, 22);
                ok = false;
            }
            ml1[r] = make_float2(steps > 0 && ok ? m : -INFINITY, l);
            if (ok && steps > 0) {                  // the whole warp: the load from tensor memory is the warp's, whatever a row's maximum
                tc_fence_after();
#pragma unroll
                for (int c = 0; c < HD; c += 32) {
                    uint32_t orr[32];
                    tmem_ld32(my_o + c, orr);
                    tmem_loaded(orr);
#pragma unroll
                    for (int d = 0; d < 32; d += 4)
                        *reinterpret_cast<uint4*>(xo + r * HD + ((((c + d) >> 2) ^ (r & 15)) << 2)) = make_uint4(orr[d], orr[d + 1], orr[d + 2], orr[d + 3]);
                }
            }
        }
        // (both groups are past their reads of the probabilities' buffers: their last P V has landed, or the walk has failed)
        asm volatile("bar.sync 6, 256;" ::: "memory");
        float acc[HD];
        if (g == 0) {
            const float2 o1 = ml1[r];
            const float mm = fmaxf(m, o1.x);
            const float w0 = m == -INFINITY ? 0.0f : at_ex2(m - mm), w1 = o1.x == -INFINITY ? 0.0f : at_ex2(o1.x - mm);
            if (ok) {
                tc_fence_after();
#pragma unroll
                for (int c = 0; c < HD; c += 32) {
                    uint32_t orr[32];
                    tmem_ld32(my_o + c, orr);
                    tmem_loaded(orr);
#pragma unroll
                    for (int d = 0; d < 32; d++) acc[c + d] = w0 == 0.0f ? 0.0f : __uint_as_float(orr[d]) * w0;
                }
                if (w1 != 0.0f) {
#pragma unroll
                    for (int d = 0; d < HD; d += 4) {
                        const float4 v = *reinterpret_cast<const float4*>(xo + r * HD + (((d >> 2) ^ (r & 15)) << 2));
                        acc[d] += v.x * w1; acc[d + 1] += v.y * w1; acc[d + 2] += v.z * w1; acc[d + 3] += v.w * w1;
                    }
                }
            }
            l = l * w0 + o1.y * w1;
            m = mm;
        }
        if (n_parts == 1) {
            if (g == 0 && ok && valid) {
                const float inv = 1.0f / l;
                __nv_bfloat16* dst = out + ((size_t)(tok0 + r) * nh + h) * HD;
#pragma unroll
                for (int d = 0; d < HD; d += 8) {
                    uint4 v;
                    v.x = at_pack(acc[d] * inv, acc[d + 1] * inv);
                    v.y = at_pack(acc[d + 2] * inv, acc[d + 3] * inv);
                    v.z = at_pack(acc[d + 4] * inv, acc[d + 5] * inv);
                    v.w = at_pack(acc[d + 6] * inv, acc[d + 7] * inv);
                    *reinterpret_cast<uint4*>(dst + d) = v;
                }
            }
        } else {
            // this part's unnormalised output, reference maximum and sum (a row without a counted key in this part leaves
            // maximum -inf and nothing else); then the parts meet as above, each group adding 32 of a row's columns
            const size_t slot = ((size_t)tile * nh + h) * sc.parts + part;
            if (g == 0 && ok && valid) {
                float* po = sc.part_o + (slot * AT_BM + r) * HD;
#pragma unroll
                for (int d = 0; d < HD; d += 4) *reinterpret_cast<float4*>(po + d) = make_float4(acc[d], acc[d + 1], acc[d + 2], acc[d + 3]);
                *reinterpret_cast<float2*>(sc.part_ml + (slot * AT_BM + r) * 2) = make_float2(m, l);
            }
            asm volatile("bar.sync 5, 256;" ::: "memory");
            if (threadIdx.x == 0) {
                int* counter = sc.counters + (size_t)tile * nh + h;
                int old;
                asm volatile("atom.acq_rel.gpu.global.add.s32 %0, [%1], 1;" : "=r"(old) : "l"(counter) : "memory");
                is_last = old == n_parts - 1;
                if (is_last) *counter = 0;
            }
            asm volatile("bar.sync 5, 256;" ::: "memory");
            if (is_last && valid) {
                const int half = g;
                const size_t first = ((size_t)tile * nh + h) * sc.parts;
                float mm = -INFINITY, ll = 0.0f, a2[32];
#pragma unroll
                for (int d = 0; d < 32; d++) a2[d] = 0.0f;
                for (int j = 0; j < n_parts; j++) {
                    const float2 ml = __ldcg(reinterpret_cast<const float2*>(sc.part_ml + ((first + j) * AT_BM + r) * 2));
                    if (ml.x == -INFINITY) continue;
                    const float cm = fmaxf(mm, ml.x);
                    const float keep = mm == -INFINITY ? 0.0f : at_ex2(mm - cm), w = at_ex2(ml.x - cm);
                    const float4* src = reinterpret_cast<const float4*>(sc.part_o + ((first + j) * AT_BM + r) * HD + half * 32);
                    ll = ll * keep + ml.y * w;
#pragma unroll
                    for (int d = 0; d < 32; d += 4) {
                        const float4 v = __ldcg(src + d / 4);
                        a2[d] = a2[d] * keep + v.x * w; a2[d + 1] = a2[d + 1] * keep + v.y * w;
                        a2[d + 2] = a2[d + 2] * keep + v.z * w; a2[d + 3] = a2[d + 3] * keep + v.w * w;
                    }
                    mm = cm;
                }
                const float inv = 1.0f / ll;
                __nv_bfloat16* dst = out + ((size_t)(tok0 + r) * nh + h) * HD + half * 32;
#pragma unroll
                for (int d = 0; d < 32; d += 8) {
                    uint4 v;
                    v.x = at_pack(a2[d] * inv, a2[d + 1] * inv);
                    v.y = at_pack(a2[d + 2] * inv, a2[d + 3] * inv);
                    v.z = at_pack(a2[d + 4] * inv, a2[d + 5] * inv);
                    v.w = at_pack(a2[d + 6] * inv, a2[d + 7] * inv);
                    *reinterpret_cast<uint4*>(dst + d) = v;
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 9) {
        if (failed) __nanosleep(200000);
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_s), "r"(TMEM_COLS) : "memory");
    }
}

// A [rows, cols] bfloat16 matrix with row stride ld (elements), read in boxes of box_rows x 64 columns, 128-byte swizzle.
static bool at_make_map(CUtensorMap* map, const void* base, long long rows, int cols, long long ld, int box_rows) {
    EncodeTiledFn enc = encode_tiled();
    if (!enc) return false;
    cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
    cuuint32_t box[2] = {64u, (cuuint32_t)box_rows};
    cuuint32_t elem[2] = {1, 1};
    return enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE,
               CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace vk

using namespace vk;

// Which of the two kernels a launch takes: 0 the first, 1 the one with two streams, 2 (default) by the size of the launch.
static int g_prefill_streams_mode = -1;
static int prefill_streams_mode() {
    if (g_prefill_streams_mode < 0) {
        const char* e = getenv("VITNA_ATT_STREAMS");
        g_prefill_streams_mode = e ? (atoi(e) ? 1 : 0) : 2;
    }
    return g_prefill_streams_mode;
}
// Returns the mode that was in force.
VK_API int vk_set_prefill_streams(int mode) {
    const int was = prefill_streams_mode();
    if (mode >= 0 && mode <= 2) g_prefill_streams_mode = mode;
    return was;
}

// Bytes of scratch for launches of up to cap_tiles tiles whose contexts reach max_context positions: the parts' outputs,
// their maxima and sums, and the counters, in that order, each 256-byte aligned.
VK_API size_t vk_attention_prefill_tcgen05_scratch_bytes(int cap_tiles, int nh, int max_context) {
    const size_t parts = (size_t)((max_context - 1) / AT_BN) / AT_PART + 1;
    auto up = [](size_t b) { return (b + 255) / 256 * 256; };
    return up((size_t)cap_tiles * nh * parts * AT_BM * 64 * 4) + up((size_t)cap_tiles * nh * parts * AT_BM * 2 * 4) +
           up((size_t)cap_tiles * nh * 4);
}

// q [n_tokens, nh*hd] bfloat16; cache [pages][2][nkv][page_size][hd] bfloat16 (one layer); tiles [n_tiles][4] with up to 128
// rows a tile; out as q.  hd = 64; page_size a multiple of 8 that divides 64 or is a multiple of it.
// scratch: vk_attention_prefill_tcgen05_scratch_bytes(cap_tiles, nh, max_context) bytes whose counters part (the last) was
// zero before the first launch; cap_tiles and max_context fix its layout; grid_context (<= max_context) bounds every
// position + 1 of this launch and sizes the grid (a captured graph keeps it).
// error: a word the kernel sets (non-zero) if a bounded wait ran out.  VK_BAD_SHAPE for what this kernel does not take.
VK_API int vk_attention_prefill_tcgen05(const void* q, const void* cache, const int32_t* block_tables, const int32_t* tiles, void* out,
                                        int n_tokens, int n_tiles, int pages, int nh, int nkv, int hd, int page_size, int max_blocks,
                                        float scale, int window, void* scratch, int cap_tiles, int max_context, int grid_context,
                                        int* error, cudaStream_t stream) {
    if (n_tiles <= 0) return VK_OK;
    if (nh <= 0 || nkv <= 0 || nh % nkv != 0 || page_size <= 0 || max_blocks <= 0 || window < 0 || n_tokens <= 0 || pages <= 0 || !error ||
        !scratch || max_context <= 0 || grid_context <= 0 || grid_context > max_context)
        return VK_BAD_SHAPE;
    if (hd != 64 || page_size % 8 != 0 || (AT_BN % page_size != 0 && page_size % AT_BN != 0)) return VK_BAD_SHAPE;
    if (nh > 65535 || n_tiles > cap_tiles) return VK_TOO_LARGE;
    const long long cache_rows = (long long)pages * 2 * nkv * page_size;
    if (cache_rows >= (1ll << 31)) return VK_TOO_LARGE;
    if (((uintptr_t)q % 16) || ((uintptr_t)cache % 16) || ((uintptr_t)out % 16) || ((uintptr_t)scratch % 16)) return VK_BAD_ALIGNMENT;
    CUtensorMap mq, mkv;
    if (!at_make_map(&mq, q, n_tokens, nh * hd, (long long)nh * hd, AT_BM)) return VK_BAD_SHAPE;
    if (!at_make_map(&mkv, cache, cache_rows, hd, hd, page_size < AT_BN ? page_size : AT_BN)) return VK_BAD_SHAPE;
    const size_t max_parts = (size_t)((max_context - 1) / AT_BN) / AT_PART + 1;
    auto up = [](size_t b) { return (b + 255) / 256 * 256; };
    AtScratch sc;
    sc.part_o = (float*)scratch;
    sc.part_ml = (float*)((char*)scratch + up((size_t)cap_tiles * nh * max_parts * AT_BM * 64 * 4));
    sc.counters = (int*)((char*)sc.part_ml + up((size_t)cap_tiles * nh * max_parts * AT_BM * 2 * 4));
    // Walks are cut only when the launch has fewer blocks than three quarters of the multiprocessors (a portion of a few
    // hundred tokens far into a context): measured, a part costs about five key steps of set-up, meeting and adding
    // up, which a whole prompt's launch (a block or more a multiprocessor already) does not win back.
    // VITNA_ATT_PART=n (n >= 16) cuts every launch into parts of n steps, for measurements.
    static const int forced = [] { const char* e = getenv("VITNA_ATT_PART"); const int v = e ? atoi(e) : 0; return v >= AT_PART ? v : 0; }();
    const bool cut = forced || (long long)n_tiles * nh * 4 <= (long long)148 * 3;
    sc.part_steps = forced ? forced : cut ? AT_PART : (1 << 24);      // never below AT_PART: the scratch is laid out for that
    sc.parts = cut ? ((grid_context - 1) / AT_BN) / sc.part_steps + 1 : 1;
    sc.n_tiles = n_tiles;
    if ((long long)n_tiles * sc.parts * nh > 0x7fffffffll) return VK_TOO_LARGE;
    // Which kernel: the one with two streams of key steps wherever a multiprocessor gets one or two blocks (measured at 9 to
    // 32 heads and 300 to 8,192 tokens: 12.7 against 13.6, 29.6 against 36.5, 32.1 against 43.0, 58.3 against 80.7
    // microseconds); from about two and a half blocks a multiprocessor on, two blocks of the first kernel that share a
    // multiprocessor keep it a little busier (50.0 against 52.0, 63.0 against 65.2, 649 against 692).
    // VITNA_ATT_STREAMS=0 / 1 in the environment, or vk_set_prefill_streams, forces one or the other (tests, measurements).
    const int forced_kernel = prefill_streams_mode();
    const long long blocks = (long long)n_tiles * sc.parts * nh;
    if (forced_kernel == 1 || (forced_kernel == 2 && blocks < 370)) {
        const size_t smem2 = (size_t)AT_BM * 64 * 2 + 2 * AS_STAGES * AT_BN * 64 * 2 + 4 * AT_BM * AT_BN * 2 + 1024 + 256;
        auto kern2 = attention_prefill_streams_kernel<64>;
        cudaError_t e2 = cudaFuncSetAttribute(kern2, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem2);
        if (e2 != cudaSuccess) return (int)e2;
        return launch_plain(kern2, dim3((unsigned)blocks), dim3(AS_THREADS), smem2, stream, mq, mkv, block_tables, tiles, (__nv_bfloat16*)out,
                            nh, nkv, page_size, max_blocks, scale, window, wait_ctl(error, WAIT_FAMILY_ATTENTION_PREFILL), sc);
    }
    const bool dbuf = false;                                // (two buffers of probabilities: measured no better than the other kernel)
    const size_t smem = (size_t)AT_BM * 64 * 2 + 2 * AT_STAGES * AT_BN * 64 * 2 + (dbuf ? 4 : 2) * AT_BM * AT_BN * 2 + 1024 + 256;
    auto kern = attention_prefill_tcgen05_kernel<64, false>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    // (an ordinary launch: started under programmatic dependent launch, with the kernel after it fetching its weights
    // meanwhile, a 2,048-token prompt at the 135M sizes took 2.90 instead of 2.72 ms)
    return launch_plain(kern, dim3(n_tiles * sc.parts * nh), dim3(AT_THREADS), smem, stream, mq, mkv, block_tables, tiles, (__nv_bfloat16*)out, nh,
                        nkv, page_size, max_blocks, scale, window, wait_ctl(error, WAIT_FAMILY_ATTENTION_PREFILL), sc);
}
