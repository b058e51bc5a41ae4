// Split-key decode attention in bfloat16 for large launches: persistent warps that stream the cache through TMA.
//
// Same decomposition, scratch and result as attention_decode_mma.cu: a unit of work is a token, a tile of up to 16
// query heads that share a key-value head, and a split of 256 keys at absolute positions; every unit leaves an
// unnormalised partial (maximum, sum, sum of p*v) and the unit that arrives last for its (token, head tile) folds the
// partials in split order.  What differs is who does a unit and how the keys arrive:
//
//   * one block a multiprocessor, twelve warps, and every WARP works through whole units by itself: the split's keys
//     in chunks of 32 with a running maximum, sum and output (the online softmax), so that no two warps ever have to
//     meet; unit u of the launch goes to warp (u mod warps of the grid), interleaved over the blocks;
//   * a chunk's keys and values come as TMA boxes straight from the pages (a box is the rows of one page for one
//     key-value head, 128-byte swizzle), issued by the warp's own lanes into the warp's own ring of two 8 KB
//     stages, each with an mbarrier; the ring runs across units, so the first chunk of the next unit is on
//     its way while the last of this one is used, and a multiprocessor always has copies in flight.
//
// A warp asks for the first chunks of its first unit before the wait on the kernel before this launch (programmatic
// dependent launch): that kernel writes the tokens' own keys and values only, and a chunk that ends before the token's
// position holds keys of earlier steps.
//
// The arithmetic of a chunk is kept short, because a warp that works alone cannot hide its own latencies: scores and
// probabilities are kept in base 2 (the scale carries log2 e, 2^x is one instruction of the special-function unit),
// keys are masked only in chunks that touch the position or the window's edge, and the running output is rescaled
// only when a chunk raises a row's maximum.
//
// Launches whose head groups have at most eight heads take the kernel's FEW form, which halves that arithmetic again:
// the chunk's keys are the 16 rows of the products and the heads the 8 columns.
//
// The separate launch-per-unit kernel leaves the memory pipe idle while a block sets up, meets and counts; here the
// copies never stop.  Chosen for head size 64 and launches with at least half as many units as the grid has
// warps; smaller launches keep the kernel that puts eight warps on one unit.
//
// A row's result does not depend on what else is in the batch: splits and chunks lie at absolute positions and the
// order of every sum is the unit's own.  Every wait on an mbarrier is bounded (see tcgen05_common.cuh).
#include "tcgen05_common.cuh"

namespace vk {

constexpr int DT_WARPS = 12, DT_THREADS = DT_WARPS * 32, DT_STAGES = 2, DT_CHUNK = 32, DT_SPLIT = 256, DT_ROWS = 16, DT_HD = 64;
constexpr int DT_CHUNKS = DT_SPLIT / DT_CHUNK;
constexpr uint32_t DT_HALF_BYTES = DT_CHUNK * DT_HD * 2, DT_STAGE_BYTES = 2 * DT_HALF_BYTES;      // keys, then values
constexpr int DT_MAX_TOKENS = 256;

struct DtArgs {
    const __nv_bfloat16* q;
    const int32_t* block_tables;
    const int32_t* token_seg;
    const int32_t* positions;
    const int32_t* tok_list;
    __nv_bfloat16* out;
    float* part_o;
    float* part_ml;
    int* counters;
    int n_tokens, nh, nkv, page_size, max_blocks, max_splits, grid_splits, counter_tiles;
    float scale;
    int window;
};

// One unit of work, from the step's metadata.
struct DtUnit {
    int zi, t, y, kvh, h0, gt, pos, lo, split, first_split, n_active, k0, c0, c1;     // chunks c0 .. c1 of the split hold counted keys
    const int32_t* bt;
};

__device__ __forceinline__ void dt_ldsm_x4(uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3, uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void dt_ldsm_x4_trans(uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3, uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void dt_mma(float* d, const uint32_t* a, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ float dt_ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ uint32_t dt_movmatrix_trans(uint32_t x) {
    uint32_t y;
    asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(y) : "r"(x));
    return y;
}
__device__ __forceinline__ uint32_t dt_pack(float x, float y) {
    __nv_bfloat162 v = __floats2bfloat162_rn(x, y);
    return *reinterpret_cast<uint32_t*>(&v);
}
// Row r (a key of the chunk), 16-byte piece j of a 128-byte row, as TMA's 128-byte swizzle lays it down.
__device__ __forceinline__ uint32_t dt_sw(uint32_t base, int row, int piece) { return base + row * 128 + ((piece ^ (row & 7)) << 4); }

// FEW: every tile has at most eight heads (a group of at most eight), and the products are turned over as in
// attention_decode_mma.cu: the chunk's keys are the 16 rows and the heads the 8 columns, S^T = K Q^T and O^T = V^T P^T,
// the probabilities transposed in registers (movmatrix) on their way into the 8-column operand.  Half the products
// and exponentials of a chunk, and half the registers for the queries and the running output.
template <bool FEW>
__global__ void __launch_bounds__(DT_THREADS, 1) attention_decode_tma_kernel(const __grid_constant__ CUtensorMap map_kv, const DtArgs a,
                                                                             const WaitCtl wc) {
    typedef __nv_bfloat16 T;
    constexpr int HD = DT_HD, KSTEPS = HD / 16, DBLK = HD / 8;
    constexpr int QR = FEW ? 2 : 4, OB = FEW ? HD / 16 : HD / 8;      // registers of a k-step's queries; blocks of the running output
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + DT_WARPS * DT_STAGES * DT_STAGE_BYTES);      // [warps][stages]
    int* ubase = reinterpret_cast<int*>(bars + DT_WARPS * DT_STAGES);                                // [n_tokens + 1]: units before token i
    __shared__ int failed;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int gq = lane >> 2, qd = lane & 3;
    const int g = a.nh / a.nkv, tiles_per_kv = (g + DT_ROWS - 1) / DT_ROWS, tiles = a.nkv * tiles_per_kv;
    const int ps = a.page_size;
    const float scale_log2 = a.scale * 1.4426950408889634f;         // scores and maxima are kept in base 2
    const int box_rows = ps < DT_CHUNK ? ps : DT_CHUNK, boxes = DT_CHUNK / box_rows;

    // ---- set-up, from the step's metadata (which no kernel of the step writes) ------------------------------------
    if (tid == 0) {
        failed = 0;
        for (int i = 0; i < DT_WARPS * DT_STAGES; i++) mbar_init(&bars[i], 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    for (int i = tid; i < a.n_tokens; i += DT_THREADS) {
        const int t = a.tok_list ? a.tok_list[i] : i;
        const int pos = a.positions[t];
        const int lo = (a.window > 0 && pos - a.window + 1 > 0) ? pos - a.window + 1 : 0;
        const int last = min(pos / DT_SPLIT, a.grid_splits - 1);          // only splits the launch was sized for (see attention_decode.cu)
        ubase[i + 1] = (last - lo / DT_SPLIT + 1) * tiles;
    }
    __syncthreads();
    if (tid == 0) {
        int run = 0;
        ubase[0] = 0;
        for (int i = 1; i <= a.n_tokens; i++) { run += ubase[i]; ubase[i] = run; }
    }
    __syncthreads();
    const int n_units = ubase[a.n_tokens];
    const int grid_warps = gridDim.x * DT_WARPS, my_first = warp * gridDim.x + blockIdx.x;     // interleaved over the blocks

    auto unit_of = [&](int u) -> DtUnit {
        DtUnit it;
        int lo_i = 0, hi_i = a.n_tokens;                  // the token whose range of units holds u
        while (hi_i - lo_i > 1) {
            const int mid = (lo_i + hi_i) >> 1;
            if (ubase[mid] <= u) lo_i = mid; else hi_i = mid;
        }
        it.zi = lo_i;
        it.t = a.tok_list ? a.tok_list[it.zi] : it.zi;
        it.pos = a.positions[it.t];
        it.lo = (a.window > 0 && it.pos - a.window + 1 > 0) ? it.pos - a.window + 1 : 0;
        it.first_split = it.lo / DT_SPLIT;
        it.n_active = min(it.pos / DT_SPLIT, a.grid_splits - 1) - it.first_split + 1;
        const int r = u - ubase[it.zi];
        it.y = r / it.n_active;
        it.split = it.first_split + r % it.n_active;
        it.kvh = it.y / tiles_per_kv;
        it.h0 = it.kvh * g + (it.y % tiles_per_kv) * DT_ROWS;
        it.gt = min(DT_ROWS, it.kvh * g + g - it.h0);
        it.k0 = it.split * DT_SPLIT;
        it.c0 = it.lo > it.k0 ? (it.lo - it.k0) / DT_CHUNK : 0;
        it.c1 = min(DT_CHUNKS - 1, (it.pos - it.k0) / DT_CHUNK);
        it.bt = a.block_tables + (size_t)a.token_seg[it.t] * a.max_blocks;
        return it;
    };

    uint8_t* my_stages = smem + (size_t)warp * DT_STAGES * DT_STAGE_BYTES;
    uint64_t* my_bars = bars + warp * DT_STAGES;

    int ipages = 0;                             // the pages of the unit the issuing cursor is in (lane j: the j-th of its split)
    // The chunk `c` of unit `it` into stage `s`: lane b asks for box b of the keys and of the values.
    auto issue = [&](const DtUnit& it, int c, int s) {
        const int kc0 = it.k0 + c * DT_CHUNK;
        int nb = (it.pos - kc0) / box_rows + 1;              // boxes whose first key is not after the position
        nb = nb < boxes ? nb : boxes;
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");      // the stage's last readers were this warp's own lanes
        if (lane == 0) mbar_expect_tx(&my_bars[s], (uint32_t)nb * box_rows * HD * 2 * 2);
        __syncwarp();
        // the page of box `lane`: the split's pages were read once, lane j holding the j-th of them (see load_pages)
        const int key = kc0 + lane * box_rows;
        const int page = __shfl_sync(0xffffffffu, ipages, key / ps - it.k0 / ps);
        if (lane < nb) {
            const int off = key % ps;
            uint8_t* dst = my_stages + (size_t)s * DT_STAGE_BYTES + lane * box_rows * (HD * 2);
            tma_load_2d(dst, &map_kv, 0, (page * 2 * a.nkv + it.kvh) * ps + off, &my_bars[s]);
            tma_load_2d(dst + DT_HALF_BYTES, &map_kv, 0, ((page * 2 + 1) * a.nkv + it.kvh) * ps + off, &my_bars[s]);
        }
    };
    // The pages of a unit's split (at most 32: pages hold at least 8 keys), lane j the j-th, in one trip: a trip to the
    // block table for every chunk would stand between the warp and its next copy.
    auto load_pages = [&](const DtUnit& it) -> int {
        const int pg0 = it.k0 / ps, pg_end = min(it.pos, it.k0 + DT_SPLIT - 1) / ps;      // the split's pages that the request has
        return pg0 + lane <= pg_end ? it.bt[pg0 + lane] : 0;
    };
    // The queries of the unit's heads as the 16-row operand: lane (gq, qd) holds rows gq and gq+8.
    // (FEW: as the 8-column operand, lane (gq, qd) holds head gq, dims 2qd, 2qd+1 and +8 of each k-step.)
    auto load_q = [&](const DtUnit& it, uint32_t (*qf)[QR]) {
        const T* r0 = a.q + ((size_t)it.t * a.nh + it.h0 + gq) * HD + 2 * qd;
        const T* r1 = r0 + (size_t)8 * HD;
        const bool on0 = gq < it.gt, on1 = gq + 8 < it.gt;
#pragma unroll
        for (int ks = 0; ks < KSTEPS; ks++) {
            if constexpr (FEW) {
                qf[ks][0] = on0 ? *reinterpret_cast<const uint32_t*>(r0 + ks * 16) : 0u;
                qf[ks][1] = on0 ? *reinterpret_cast<const uint32_t*>(r0 + ks * 16 + 8) : 0u;
            } else {
                qf[ks][0] = on0 ? *reinterpret_cast<const uint32_t*>(r0 + ks * 16) : 0u;
                qf[ks][1] = on1 ? *reinterpret_cast<const uint32_t*>(r1 + ks * 16) : 0u;
                qf[ks][2] = on0 ? *reinterpret_cast<const uint32_t*>(r0 + ks * 16 + 8) : 0u;
                qf[ks][3] = on1 ? *reinterpret_cast<const uint32_t*>(r1 + ks * 16 + 8) : 0u;
            }
        }
    };

    // ---- the stream of chunks: an issuing cursor runs up to DT_STAGES chunks (and at most one unit) ahead --------
    const bool have = my_first < n_units;
    int iu = my_first;                          // unit being issued, and its next chunk
    DtUnit iunit = have ? unit_of(iu) : DtUnit{};
    int ic = iunit.c0;
    uint32_t qn[KSTEPS][QR];                    // the queries of the unit the issuing cursor has reached
    int issued = 0, consumed = 0;               // chunks so far: stage = count % DT_STAGES, parity = (count / DT_STAGES) & 1
    int cu = my_first;                          // unit being consumed
    bool ok = true;
    // The first chunks of the warp's first unit are asked for before the wait on the kernel before this one, which
    // writes the token's own key and value only: every chunk that ends before the token's position holds keys of
    // earlier steps.
    if (have) {
        ipages = load_pages(iunit);
        while (issued < DT_STAGES && ic <= iunit.c1 && iunit.k0 + ic * DT_CHUNK + DT_CHUNK - 1 < iunit.pos) {
            issue(iunit, ic, issued % DT_STAGES);
            issued++;
            ic++;
        }
    }
    dependency_wait();                          // q and the token's own key and value come from the kernel before this one
    let_dependents_start();
    if (!have) return;
    load_q(iunit, qn);

    // The issuing cursor stops before the unit after next (its queries would overwrite, in qn, those of a unit not yet
    // begun); iu then names that unit without its fields, which are made when the cursor may go on.
    bool ipending = false;
    auto next_unit = [&]() {                    // the issuing cursor has passed its unit's last chunk
        iu += grid_warps;
        if (iu >= n_units) return;
        if (iu > cu + grid_warps) { ipending = true; return; }
        iunit = unit_of(iu);
        ic = iunit.c0;
        load_q(iunit, qn);
        ipages = load_pages(iunit);
    };
    if (ic > iunit.c1) next_unit();             // (a first unit of one or two chunks, none at the position, is asked for whole)

    while (cu < n_units && ok) {
        const DtUnit it = cu == iu && !ipending ? iunit : unit_of(cu);
        uint32_t qf[KSTEPS][QR];
        if (cu == iu && !ipending) {
#pragma unroll
            for (int ks = 0; ks < KSTEPS; ks++) {
#pragma unroll
                for (int r = 0; r < QR; r++) qf[ks][r] = qn[ks][r];
            }
        } else {
            load_q(it, qf);                     // the issuing cursor is past this unit: its queries are gone from qn
        }
        float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.0f, 0.0f};
        float o[OB][4];
#pragma unroll
        for (int db = 0; db < OB; db++) { o[db][0] = o[db][1] = o[db][2] = o[db][3] = 0.0f; }

        for (int c = it.c0; c <= it.c1 && ok; c++) {
            // keep the ring full
            if (ipending && iu <= cu + grid_warps && iu < n_units) {
                iunit = unit_of(iu);
                ic = iunit.c0;
                load_q(iunit, qn);
                ipages = load_pages(iunit);
                ipending = false;
            }
            while (!ipending && issued - consumed < DT_STAGES && iu < n_units) {
                issue(iunit, ic, issued % DT_STAGES);
                issued++;
                if (++ic > iunit.c1) {
                    next_unit();
                    if (iu >= n_units || ipending) break;
                }
            }
            const int s = consumed % DT_STAGES;
            if (!__all_sync(0xffffffffu, mbar_wait(&my_bars[s], (consumed / DT_STAGES) & 1, wc.cycles))) {
                if (lane == 0) give_up(wc.error, &failed, 41);
                ok = false;
                break;
            }
            const uint32_t kbase = smem_u32(my_stages + (size_t)s * DT_STAGE_BYTES), vbase = kbase + DT_HALF_BYTES;
            const int kc0 = it.k0 + c * DT_CHUNK;
            // values of rows that hold no counted key (beyond the position: slots not yet written, boxes not asked for)
            // are never counted, but 0 * garbage must not be NaN
            const int nvalid = min(DT_CHUNK, it.pos - kc0 + 1);
            if (nvalid < DT_CHUNK) {
                uint8_t* vs = my_stages + (size_t)s * DT_STAGE_BYTES + DT_HALF_BYTES;
                for (int i = lane; i < (DT_CHUNK - nvalid) * 8; i += 32)
                    *reinterpret_cast<uint4*>(vs + (nvalid + i / 8) * 128 + (i & 7) * 16) = make_uint4(0, 0, 0, 0);
                __syncwarp();
            }

            const bool edge = kc0 + DT_CHUNK - 1 > it.pos || kc0 < it.lo;
            if constexpr (FEW) {
                // ---- scores: two blocks of 16 keys; lane (gq, qd) gets keys gq and gq+8 of a block for heads 2qd, 2qd+1 ----
                float sc[2][4];
#pragma unroll
                for (int kb = 0; kb < 2; kb++) {
                    sc[kb][0] = sc[kb][1] = sc[kb][2] = sc[kb][3] = 0.0f;
#pragma unroll
                    for (int ks = 0; ks < KSTEPS; ks++) {
                        uint32_t af[4];
                        dt_ldsm_x4(af[0], af[1], af[2], af[3], dt_sw(kbase, kb * 16 + (lane & 15), ks * 2 + (lane >> 4)));
                        dt_mma(sc[kb], af, qf[ks][0], qf[ks][1]);
                    }
                }
                float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
                for (int kb = 0; kb < 2; kb++) {
#pragma unroll
                    for (int e = 0; e < 4; e++) {
                        float v = sc[kb][e] * scale_log2;
                        if (edge) {
                            const int kk = kc0 + kb * 16 + gq + (e >> 1) * 8;
                            if (!(kk <= it.pos && kk >= it.lo)) v = -INFINITY;
                        }
                        sc[kb][e] = v;
                        mx[e & 1] = fmaxf(mx[e & 1], v);
                    }
                }
#pragma unroll
                for (int h = 0; h < 2; h++) {           // over the eight lanes that hold the head's other keys; finite as below
                    mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 4));
                    mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 8));
                    mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 16));
                }
                if (__any_sync(0xffffffffu, mx[0] > m_run[0] || mx[1] > m_run[1])) {
                    float alpha[2];
#pragma unroll
                    for (int h = 0; h < 2; h++) {
                        const float m_new = fmaxf(m_run[h], mx[h]);
                        alpha[h] = dt_ex2(m_run[h] - m_new);        // 0 for the unit's first chunk
                        m_run[h] = m_new;
                        l_run[h] *= alpha[h];
                    }
#pragma unroll
                    for (int hb = 0; hb < OB; hb++) { o[hb][0] *= alpha[0]; o[hb][1] *= alpha[1]; o[hb][2] *= alpha[0]; o[hb][3] *= alpha[1]; }
                }
                uint32_t ph[2][2], pl[2][2];            // the 8-column operand of the two blocks of 16 keys, high and low parts
#pragma unroll
                for (int kb = 0; kb < 2; kb++) {
#pragma unroll
                    for (int half = 0; half < 2; half++) {      // keys gq (0) and gq+8 (1) of the block
                        const float p0 = dt_ex2(sc[kb][2 * half] - m_run[0]), p1 = dt_ex2(sc[kb][2 * half + 1] - m_run[1]);
                        l_run[0] += p0;                 // this lane's share of the heads' sums; the lanes meet at the unit's end
                        l_run[1] += p1;
                        const __nv_bfloat162 hv = __floats2bfloat162_rn(p0, p1);
                        // [key][heads 2qd, 2qd+1] -> [head][keys 2qd, 2qd+1]: what the 8-column operand wants
                        ph[kb][half] = dt_movmatrix_trans(*reinterpret_cast<const uint32_t*>(&hv));
                        pl[kb][half] = dt_movmatrix_trans(dt_pack(p0 - __bfloat162float(hv.x), p1 - __bfloat162float(hv.y)));
                    }
                }
                // ---- O^T += V^T P^T: blocks of 16 dims; lane (gq, qd) gets dims gq and gq+8 of a block for heads 2qd, 2qd+1 ----
#pragma unroll
                for (int kb = 0; kb < 2; kb++) {
#pragma unroll
                    for (int hb = 0; hb < OB; hb++) {
                        uint32_t af[4];
                        dt_ldsm_x4_trans(af[0], af[1], af[2], af[3], dt_sw(vbase, kb * 16 + (lane & 7) + ((lane >> 4) << 3), hb * 2 + ((lane >> 3) & 1)));
                        dt_mma(o[hb], af, ph[kb][0], ph[kb][1]);
                        dt_mma(o[hb], af, pl[kb][0], pl[kb][1]);
                    }
                }
            } else {
                // ---- scores of the chunk's 32 keys: four blocks of 8 keys ----------------------------------------------
                float sc[4][4];
#pragma unroll
                for (int nb = 0; nb < 4; nb++) { sc[nb][0] = sc[nb][1] = sc[nb][2] = sc[nb][3] = 0.0f; }
#pragma unroll
                for (int ks = 0; ks < KSTEPS; ks++) {
#pragma unroll
                    for (int nb2 = 0; nb2 < 2; nb2++) {
                        uint32_t b0, b1, b2, b3;
                        dt_ldsm_x4(b0, b1, b2, b3, dt_sw(kbase, nb2 * 16 + (lane & 7) + ((lane >> 4) << 3), ks * 2 + ((lane >> 3) & 1)));
                        dt_mma(sc[nb2 * 2], qf[ks], b0, b1);
                        dt_mma(sc[nb2 * 2 + 1], qf[ks], b2, b3);
                    }
                }
                // scale (base 2) and, in a chunk that touches the position or the window's edge, mask; rows gq and gq+8
                // (heads), keys kc0 + nb*8 + 2*qd + {0,1}
                float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
                for (int nb = 0; nb < 4; nb++) {
#pragma unroll
                    for (int e = 0; e < 4; e++) {
                        float v = sc[nb][e] * scale_log2;
                        if (edge) {
                            const int kk = kc0 + nb * 8 + qd * 2 + (e & 1);
                            if (!(kk <= it.pos && kk >= it.lo)) v = -INFINITY;
                        }
                        sc[nb][e] = v;
                        mx[e >> 1] = fmaxf(mx[e >> 1], v);
                    }
                }
#pragma unroll
                for (int r = 0; r < 2; r++) {           // finite: the chunk has at least one key that every row counts
                    mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
                    mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
                }
                if (__any_sync(0xffffffffu, mx[0] > m_run[0] || mx[1] > m_run[1])) {
                    // a row's maximum rises (always in the unit's first chunk): what has been summed so far is rescaled
                    float alpha[2];
#pragma unroll
                    for (int r = 0; r < 2; r++) {
                        const float m_new = fmaxf(m_run[r], mx[r]);
                        alpha[r] = dt_ex2(m_run[r] - m_new);        // 0 for the unit's first chunk
                        m_run[r] = m_new;
                        l_run[r] *= alpha[r];
                    }
#pragma unroll
                    for (int db = 0; db < DBLK; db++) { o[db][0] *= alpha[0]; o[db][1] *= alpha[0]; o[db][2] *= alpha[1]; o[db][3] *= alpha[1]; }
                }
                uint32_t ph[2][4], pl[2][4];            // the 16-row operand of the two k-steps of 16 keys, high and low parts
#pragma unroll
                for (int nb = 0; nb < 4; nb++) {
                    const float p0 = dt_ex2(sc[nb][0] - m_run[0]), p1 = dt_ex2(sc[nb][1] - m_run[0]);
                    const float p2 = dt_ex2(sc[nb][2] - m_run[1]), p3 = dt_ex2(sc[nb][3] - m_run[1]);
                    l_run[0] += p0 + p1;                // this lane's share of the row's sum; the quad meets at the unit's end
                    l_run[1] += p2 + p3;
                    const __nv_bfloat162 h01 = __floats2bfloat162_rn(p0, p1), h23 = __floats2bfloat162_rn(p2, p3);
                    const int kk = nb >> 1, hi = (nb & 1) * 2;
                    ph[kk][hi] = *reinterpret_cast<const uint32_t*>(&h01);
                    ph[kk][hi + 1] = *reinterpret_cast<const uint32_t*>(&h23);
                    pl[kk][hi] = dt_pack(p0 - __bfloat162float(h01.x), p1 - __bfloat162float(h01.y));
                    pl[kk][hi + 1] = dt_pack(p2 - __bfloat162float(h23.x), p3 - __bfloat162float(h23.y));
                }
                // ---- p * v over the chunk's keys, all head dimensions --------------------------------------------------
#pragma unroll
                for (int kk = 0; kk < 2; kk++) {
#pragma unroll
                    for (int db = 0; db < DBLK; db += 2) {
                        uint32_t b0, b1, b2, b3;
                        dt_ldsm_x4_trans(b0, b1, b2, b3, dt_sw(vbase, kk * 16 + (lane & 15), db + (lane >> 4)));
                        dt_mma(o[db], ph[kk], b0, b1);
                        dt_mma(o[db], pl[kk], b0, b1);
                        dt_mma(o[db + 1], ph[kk], b2, b3);
                        dt_mma(o[db + 1], pl[kk], b2, b3);
                    }
                }
            }
            __syncwarp();                           // every lane is past its reads of the stage
            consumed++;
        }
        if (!ok) break;

        // ---- the unit's partial (or, for a single split, the result) --------------------------------------------
        const bool single = it.n_active == 1;
        if constexpr (FEW) {
            float l[2];
#pragma unroll
            for (int h = 0; h < 2; h++) {
                l[h] = l_run[h] + __shfl_xor_sync(0xffffffffu, l_run[h], 4);
                l[h] += __shfl_xor_sync(0xffffffffu, l[h], 8);
                l[h] += __shfl_xor_sync(0xffffffffu, l[h], 16);
            }
#pragma unroll
            for (int e = 0; e < 2; e++) {               // head 2qd + e: this lane has its dims gq and gq+8 of every block of 16
                const int row = 2 * qd + e;
                if (row >= it.gt) continue;
                if (single) {
                    const float inv = 1.0f / l[e];
                    T* dst = a.out + ((size_t)it.t * a.nh + it.h0 + row) * HD + gq;
#pragma unroll
                    for (int hb = 0; hb < OB; hb++) {
                        dst[hb * 16] = __float2bfloat16_rn(o[hb][e] * inv);
                        dst[hb * 16 + 8] = __float2bfloat16_rn(o[hb][2 + e] * inv);
                    }
                } else {
                    const size_t slot = ((size_t)it.zi * a.nh + it.h0 + row) * a.max_splits + it.split;
                    float* dst = a.part_o + slot * HD + gq;
#pragma unroll
                    for (int hb = 0; hb < OB; hb++) {
                        dst[hb * 16] = o[hb][e];
                        dst[hb * 16 + 8] = o[hb][2 + e];
                    }
                    if (gq == 0) *reinterpret_cast<float2*>(a.part_ml + slot * 2) = make_float2(m_run[e], l[e]);
                }
            }
        } else {
            float l[2];
#pragma unroll
            for (int r = 0; r < 2; r++) {
                l[r] = l_run[r] + __shfl_xor_sync(0xffffffffu, l_run[r], 1);
                l[r] += __shfl_xor_sync(0xffffffffu, l[r], 2);
            }
#pragma unroll
            for (int e = 0; e < 2; e++) {
                const int row = gq + 8 * e;
                if (row >= it.gt) continue;
                if (single) {
                    const float inv = 1.0f / l[e];
                    T* dst = a.out + ((size_t)it.t * a.nh + it.h0 + row) * HD + qd * 2;
#pragma unroll
                    for (int db = 0; db < DBLK; db++)
                        *reinterpret_cast<uint32_t*>(dst + db * 8) = dt_pack(o[db][2 * e] * inv, o[db][2 * e + 1] * inv);
                } else {
                    const size_t slot = ((size_t)it.zi * a.nh + it.h0 + row) * a.max_splits + it.split;
                    float* dst = a.part_o + slot * HD + qd * 2;
#pragma unroll
                    for (int db = 0; db < DBLK; db++) *reinterpret_cast<float2*>(dst + db * 8) = make_float2(o[db][2 * e], o[db][2 * e + 1]);
                    if (qd == 0) *reinterpret_cast<float2*>(a.part_ml + slot * 2) = make_float2(m_run[e], l[e]);
                }
            }
        }
        if (!single) {
            // The warp's partial is written; lane 0's counting releases it to the other units' warps and acquires theirs.
            __syncwarp();
            int* counter = a.counters + (size_t)it.zi * a.counter_tiles + it.y;
            int old = 0;
            if (lane == 0) {
                asm volatile("atom.acq_rel.gpu.global.add.s32 %0, [%1], 1;" : "=r"(old) : "l"(counter) : "memory");
                if (old == it.n_active - 1) *counter = 0;       // ready for the next launch
            }
            old = __shfl_sync(0xffffffffu, old, 0);
            if (old == it.n_active - 1) {
                // The last to arrive folds the splits in split order, a row at a time: a lane takes the row's output elements
                // `lane` and `lane + 32`, and asks for the maxima, sums and partial outputs of sixteen splits in one trip.
                for (int h = 0; h < it.gt; h++) {
                    const size_t row = ((size_t)it.zi * a.nh + it.h0 + h) * a.max_splits + it.first_split;
                    const float2* ml = reinterpret_cast<const float2*>(a.part_ml) + row;
                    const float* po = a.part_o + row * HD + lane;
                    float mm = -INFINITY, ll = 0.0f, o0 = 0.0f, o1 = 0.0f;
                    for (int j0 = 0; j0 < it.n_active; j0 += 16) {
                        float2 st[16];
                        float p0[16], p1[16];
#pragma unroll
                        for (int j = 0; j < 16; j++) {
                            const bool on = j0 + j < it.n_active;
                            st[j] = on ? __ldcg(ml + j0 + j) : make_float2(-INFINITY, 0.0f);
                            p0[j] = on ? __ldcg(po + (size_t)(j0 + j) * HD) : 0.0f;
                            p1[j] = on ? __ldcg(po + (size_t)(j0 + j) * HD + 32) : 0.0f;
                        }
                        float cm = mm;
#pragma unroll
                        for (int j = 0; j < 16; j++) cm = fmaxf(cm, st[j].x);
                        const float keep = mm == -INFINITY ? 0.0f : dt_ex2(mm - cm);       // maxima are in base 2
                        ll *= keep;
                        o0 *= keep;
                        o1 *= keep;
#pragma unroll
                        for (int j = 0; j < 16; j++) {
                            const float e = st[j].x == -INFINITY ? 0.0f : dt_ex2(st[j].x - cm);
                            ll += st[j].y * e;
                            o0 += p0[j] * e;
                            o1 += p1[j] * e;
                        }
                        mm = cm;
                    }
                    __nv_bfloat16* dst = a.out + ((size_t)it.t * a.nh + it.h0 + h) * HD + lane;
                    dst[0] = __float2bfloat16_rn(o0 / ll);
                    dst[32] = __float2bfloat16_rn(o1 / ll);
                }
            }
        }
        cu += grid_warps;
    }
    if (!ok) __nanosleep(200000);               // after a failed wait: let the copies in flight land before the block's memory goes
}

// The layer's cache as a matrix of 128-byte rows, read in boxes of box_rows rows with the 128-byte swizzle.
static bool dt_make_map(CUtensorMap* map, const void* base, long long rows, int box_rows) {
    EncodeTiledFn enc = encode_tiled();
    if (!enc) return false;
    cuuint64_t dims[2] = {(cuuint64_t)DT_HD, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)DT_HD * 2};
    cuuint32_t box[2] = {(cuuint32_t)DT_HD, (cuuint32_t)box_rows};
    cuuint32_t elem[2] = {1, 1};
    return enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE,
               CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// 0: never chosen; 1: chosen whenever it takes the sizes; 2: chosen by the size rule below.  VITNA_DECODE_TMA=0 or 1 in
// the environment sets it at start; vk_set_decode_tma changes it (tests and measurements run both kernels on the same sizes).
static int g_decode_tma_mode = -1;

static int decode_tma_mode() {
    if (g_decode_tma_mode < 0) {
        const char* e = getenv("VITNA_DECODE_TMA");
        g_decode_tma_mode = e ? (e[0] == '1' ? 1 : e[0] == '0' ? 0 : 2) : 2;
    }
    return g_decode_tma_mode;
}

// Whether launches whose head groups have at most eight heads take the kernel with the keys as rows (1, the default) or
// the one with the heads as rows (0).  VITNA_DECODE_TMA_FEW=0 in the environment, or vk_set_decode_tma_few.
static int g_decode_tma_few = -1;

static int decode_tma_few() {
    if (g_decode_tma_few < 0) {
        const char* e = getenv("VITNA_DECODE_TMA_FEW");
        g_decode_tma_few = e && e[0] == '0' ? 0 : 1;
    }
    return g_decode_tma_few;
}

// Whether this kernel takes the launch, and is the better choice for it: head size 64, pages of 8, 16 or a multiple of 32
// slots, and at least half as many units (at most: the grid's splits may not all be in use) as the grid has warps.
bool decode_tma_takes(int n_tokens, int nh, int nkv, int hd, int page_size, int pages, int grid_splits, const void* q, const void* cache,
                      const int* error) {
    const int mode = decode_tma_mode();
    if (mode == 0 || !error || pages <= 0 || hd != DT_HD || n_tokens > DT_MAX_TOKENS) return false;
    if (page_size % 8 != 0 || (DT_CHUNK % page_size != 0 && page_size % DT_CHUNK != 0)) return false;
    if (((uintptr_t)q % 4) || ((uintptr_t)cache % 16)) return false;
    if ((long long)pages * 2 * nkv * page_size >= (1ll << 31)) return false;
    const int g = nh / nkv, tiles = nkv * ((g + DT_ROWS - 1) / DT_ROWS);
    return mode == 1 || (long long)n_tokens * tiles * grid_splits >= 148 * DT_WARPS / 2;
}

int launch_decode_tma(const void* q, const void* cache, const int32_t* bt, const int32_t* token_seg, const int32_t* positions,
                      const int32_t* tok_list, void* out, float* part_o, float* part_ml, int* counters, int n_tokens, int nh, int nkv,
                      int page_size, int pages, int max_blocks, int splits, int grid_splits, int counter_tiles, float scale, int window,
                      int* error, cudaStream_t stream) {
    CUtensorMap map;
    if (!dt_make_map(&map, cache, (long long)pages * 2 * nkv * page_size, page_size < DT_CHUNK ? page_size : DT_CHUNK)) return VK_BAD_SHAPE;
    DtArgs a{(const __nv_bfloat16*)q, bt, token_seg, positions, tok_list, (__nv_bfloat16*)out, part_o, part_ml, counters,
             n_tokens, nh, nkv, page_size, max_blocks, splits, grid_splits, counter_tiles, scale, window};
    const size_t smem = (size_t)DT_WARPS * DT_STAGES * DT_STAGE_BYTES + DT_WARPS * DT_STAGES * 8 + (DT_MAX_TOKENS + 1) * 4 + 1024;
    const bool few = nh / nkv <= 8 && decode_tma_few() == 1;
    auto kern = few ? attention_decode_tma_kernel<true> : attention_decode_tma_kernel<false>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    int sms = 148, dev = 0;
    cudaGetDevice(&dev);
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) sms = 148;
    const int g = nh / nkv, tiles = nkv * ((g + DT_ROWS - 1) / DT_ROWS);
    const long long most = (long long)n_tokens * tiles * grid_splits;       // units, at most
    const int blocks = most < sms ? (int)most : sms;
    return launch_dependent(kern, dim3(blocks), dim3(DT_THREADS), smem, stream, map, a, wait_ctl(error, WAIT_FAMILY_ATTENTION_DECODE));
}

}  // namespace vk

// Which launches the persistent TMA kernel takes: 0 none, 1 all whose sizes it takes, 2 those the size rule gives it
// (the default).  Returns the mode that was in force.
// Whether head groups of at most eight take the routine with the keys as rows (1) or the general one (0).  Returns what was in force.
VK_API int vk_set_decode_tma_few(int mode) {
    const int before = vk::decode_tma_few();
    if (mode == 0 || mode == 1) vk::g_decode_tma_few = mode;
    return before;
}

VK_API int vk_set_decode_tma(int mode) {
    const int before = vk::decode_tma_mode();
    if (mode >= 0 && mode <= 2) vk::g_decode_tma_mode = mode;
    return before;
}
