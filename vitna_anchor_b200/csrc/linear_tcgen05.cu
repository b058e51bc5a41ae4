// Prompt-sized matrix products in bfloat16 on the fifth-generation tensor cores:
// out[M, N] = x[M, K] * W[N, K]^T, float32 accumulation in tensor memory.
//
// One block computes a 128 x BN tile of the output.  Warp 0 (one lane) feeds a ring of shared-memory
// stages with TMA (cp.async.bulk.tensor, 128-byte swizzle, out-of-range rows and columns read as zero);
// warp 1 (one lane) issues tcgen05.mma (M = 128, N = BN, K = 16 per instruction, both operands K-major)
// into a BN-column accumulator in tensor memory and releases stages with tcgen05.commit; warps 2-5 read
// the accumulator with tcgen05.ld, each its own 32 lanes, and store it: as bfloat16, as float32, or
// added into a float32 output (the residual sum).  No cluster, no multicast: every block loads its own
// tiles.  Each output element's sum runs over K in the same order whatever M is, so a row's result does
// not depend on the batch.
//
// Every wait on an mbarrier is bounded: after the launch's limit (about a second unless the host set another) a
// waiter sets *error (a word the host can read), the block stops issuing work, lets its copies land, frees its
// tensor memory and returns.
#include <cstdlib>

#include "tcgen05_common.cuh"

namespace vk {

constexpr int TC_BM = 128, TC_BK = 64, TC_THREADS = 192;
template <int BN> struct TcStages { static constexpr int N = BN >= 128 ? 3 : 4; };   // 96 KB of stages either way: two blocks a multiprocessor
enum { TC_SAME = 0, TC_F32 = 1, TC_ACC = 2, TC_SWIGLU = 3, TC_ROPE = 4 };

// What the fused epilogues need besides the accumulator.
//   TC_SWIGLU  the weight is [2*inter, K], gate rows then up rows; a block's tile is 64 gate rows and the 64 up rows
//              of the same columns (two TMA loads a stage), out [M, inter] = silu(gate) * up
//              (engine/src/ops.c:283-288; both rounded to bfloat16 first, as the separate kernels store them)
//   TC_ROPE    the weight is [(nh + 2*nkv) * hd, K]; BN = hd, so a tile is one head: a q head is rotated by the
//              token's position and written to out [M, nh*hd]; a k head is rotated and written into the token's
//              cache slot; a v head is written there as it is (engine/src/ops.c:273-281, engine/src/model.c:927-930)
// silu(g) * up for the bfloat16 path: 2^x and the reciprocal come from the special-function unit (relative error about
// 1e-6, far below the bfloat16 rounding of the result); the float32 path keeps expf and the division.
__device__ __forceinline__ float tc_silu_mul(float g, float up) {
    float e;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(-1.4426950408889634f * g));
    return __fdividef(g, 1.0f + e) * up;
}

struct TcExtra {
    int tma_out;                 // TC_ACC: the tile is added into out by one TMA reduction from shared memory (map_out is valid)
    int inter;
    const int32_t* positions;
    const float* cos_t;
    const float* sin_t;
    const int32_t* slot;
    __nv_bfloat16* cache;
    int nh, nkv, hd, page_size;
};

template <int BN, int EPI>
__global__ void __launch_bounds__(TC_THREADS) linear_tcgen05_kernel(const __grid_constant__ CUtensorMap map_x,
                                                                    const __grid_constant__ CUtensorMap map_w,
                                                                    const __grid_constant__ CUtensorMap map_out, void* __restrict__ out,
                                                                    int M, int N, int K, const WaitCtl wc, const TcExtra ex) {
    constexpr int TC_STAGES = TcStages<BN>::N;
    constexpr uint32_t A_BYTES = TC_BM * TC_BK * 2, B_BYTES = BN * TC_BK * 2, STAGE_BYTES = A_BYTES + B_BYTES;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + TC_STAGES * STAGE_BYTES);
    uint64_t* empty = full + TC_STAGES;
    uint64_t* acc_full = empty + TC_STAGES;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_full + 1);

    __shared__ int failed;                // set when a bounded wait of this block ran out

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int m0 = blockIdx.y * TC_BM, n0 = blockIdx.x * (EPI == TC_SWIGLU ? BN / 2 : BN);     // first output column of the tile
    const int num_kb = (K + TC_BK - 1) / TC_BK;

    if (threadIdx.x == 0) {
        failed = 0;
        for (int s = 0; s < TC_STAGES; s++) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
        mbar_init(acc_full, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(BN) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        if (lane == 0) {
            // producer: fill a stage as soon as the tensor core has released it.  The weight tiles of the first
            // stages are asked for before the wait on the kernel before this one (weights are nobody's output);
            // the activation tiles follow the wait.
            auto load_w = [&](int kb, int s) {
                if (EPI == TC_SWIGLU) {     // rows n0 .. n0+BN/2 of gate, then the same rows of up: the map's box is BN/2 rows
                    tma_load_2d(smem + s * STAGE_BYTES + A_BYTES, &map_w, kb * TC_BK, n0, &full[s]);
                    tma_load_2d(smem + s * STAGE_BYTES + A_BYTES + B_BYTES / 2, &map_w, kb * TC_BK, ex.inter + n0, &full[s]);
                } else {
                    tma_load_2d(smem + s * STAGE_BYTES + A_BYTES, &map_w, kb * TC_BK, n0, &full[s]);
                }
            };
            // (a stage named by wc.skip_stage is left unarmed and unfilled: a test of the give-up path)
            const int early = num_kb < TC_STAGES ? num_kb : TC_STAGES;
            for (int kb = 0; kb < early; kb++) {
                if (kb == wc.skip_stage) continue;
                mbar_expect_tx(&full[kb], STAGE_BYTES);
                load_w(kb, kb);
            }
            dependency_wait();
            for (int kb = 0; kb < early; kb++)
                if (kb != wc.skip_stage) tma_load_2d(smem + kb * STAGE_BYTES, &map_x, kb * TC_BK, m0, &full[kb]);
            for (int kb = early; kb < num_kb; kb++) {
                const int s = kb % TC_STAGES;
                if (!mbar_wait(&empty[s], ((kb / TC_STAGES) & 1) ^ 1, wc.cycles)) { give_up(wc.error, &failed, 1); break; }
                if (kb == wc.skip_stage) continue;
                mbar_expect_tx(&full[s], STAGE_BYTES);
                tma_load_2d(smem + s * STAGE_BYTES, &map_x, kb * TC_BK, m0, &full[s]);
                load_w(kb, s);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            const uint32_t idesc = umma_idesc_bf16(TC_BM, BN);
            const uint32_t a_lo0 = umma_desc_lo(smem_u32(smem));      // low words of the descriptors (see umma_bf16_lo)
            bool ok = true;
            for (int kb = 0; kb < num_kb && ok; kb++) {
                const int s = kb % TC_STAGES;
                if (!mbar_wait(&full[s], (kb / TC_STAGES) & 1, wc.cycles)) { give_up(wc.error, &failed, 2); ok = false; break; }
                tc_fence_after();
                const uint32_t a_lo = a_lo0 + s * (STAGE_BYTES >> 4), b_lo = a_lo + (A_BYTES >> 4);
#pragma unroll
                for (int k = 0; k < TC_BK / 16; k++) umma_bf16_lo(tmem_base, a_lo + 2 * k, b_lo + 2 * k, idesc, (kb | k) != 0);
                umma_commit(&empty[s]);           // arrives when the instructions above have read the stage
            }
            umma_commit(acc_full);                // arrives when every instruction has written the accumulator
        }
    } else {
        // epilogue: warp w reads lanes 32*(w%4) .. +31 of the accumulator, one output row per thread
        const int quarter = warp & 3;
        const int row = m0 + quarter * 32 + lane;
        dependency_wait();                 // what this block reads besides weights, and everything it writes, is after the kernel before
        let_dependents_start();
        // the residual sum's old values for the first 64 columns are read while the tensor core works
        float4 pre[2][8];
        if (EPI == TC_ACC && !ex.tma_out && row < M && (N % 4 == 0)) {
#pragma unroll
            for (int c2 = 0; c2 < 2; c2++) {
                const int col = n0 + c2 * 32;
                if (c2 * 32 < BN && col + 32 <= N) {
                    const float* o = reinterpret_cast<const float*>(out) + (size_t)row * N + col;
#pragma unroll
                    for (int j = 0; j < 8; j++) pre[c2][j] = *reinterpret_cast<const float4*>(o + 4 * j);
                }
            }
        }
        // the rotation's cosines and sines of this row's position: read while the tensor core works
        float4 rc[BN / 8], rs[BN / 8];
        if (EPI == TC_ROPE && row < M && blockIdx.x < ex.nh + ex.nkv) {
            const int p0 = ex.positions[row];
            const float4* cp = reinterpret_cast<const float4*>(ex.cos_t + (size_t)p0 * (BN / 2));
            const float4* sp = reinterpret_cast<const float4*>(ex.sin_t + (size_t)p0 * (BN / 2));
#pragma unroll
            for (int j = 0; j < BN / 8; j++) { rc[j] = cp[j]; rs[j] = sp[j]; }
        }
        bool got = mbar_wait(acc_full, 0, wc.cycles);
        if (!got && lane == 0) give_up(wc.error, &failed, 3);
        if (EPI == TC_ACC && ex.tma_out) {         // the four epilogue warps meet below: they go on together or not at all
            asm volatile("bar.sync 1, 128;" ::: "memory");
            got = *reinterpret_cast<volatile int*>(&failed) == 0;
        }
        if (!got) {
        } else if (EPI == TC_SWIGLU) {
            tc_fence_after();
            const uint32_t lane_base = tmem_base + ((uint32_t)(quarter * 32) << 16);
#pragma unroll
            for (int c = 0; c < BN / 2; c += 32) {
                uint32_t gr[32], ur[32];
                __syncwarp();
                tmem_ld32(lane_base + c, gr);
                tmem_ld32(lane_base + BN / 2 + c, ur);
                const int col = n0 + c;
                if (row < M && col < ex.inter) {
                    __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(out) + (size_t)row * ex.inter + col;
                    uint32_t packed[16];
#pragma unroll
                    for (int j = 0; j < 32; j += 2) {
                        float a[2];
#pragma unroll
                        for (int e = 0; e < 2; e++) {
                            const float gte = __bfloat162float(__float2bfloat16_rn(__uint_as_float(gr[j + e])));
                            const float up = __bfloat162float(__float2bfloat16_rn(__uint_as_float(ur[j + e])));
                            a[e] = tc_silu_mul(gte, up);
                        }
                        __nv_bfloat162 v = __floats2bfloat162_rn(a[0], a[1]);
                        packed[j / 2] = *reinterpret_cast<uint32_t*>(&v);
                    }
                    if (col + 32 <= ex.inter && (ex.inter % 8 == 0)) {
#pragma unroll
                        for (int j = 0; j < 4; j++)
                            *reinterpret_cast<uint4*>(o + 8 * j) = make_uint4(packed[4 * j], packed[4 * j + 1], packed[4 * j + 2], packed[4 * j + 3]);
                    } else {
                        for (int j = 0; j < 32 && col + j < ex.inter; j++)
                            o[j] = __ushort_as_bfloat16((unsigned short)((packed[j / 2] >> ((j & 1) * 16)) & 0xffffu));
                    }
                }
            }
        } else if (EPI == TC_ROPE) {
            tc_fence_after();
            // the tile is head number blockIdx.x: q heads, then k heads, then v heads; BN = hd
            constexpr int HALF = BN / 2;
            const uint32_t lane_base = tmem_base + ((uint32_t)(quarter * 32) << 16);
            const int head = blockIdx.x;
            const bool is_q = head < ex.nh, is_k = !is_q && head < ex.nh + ex.nkv;
            const int sl = row < M ? ex.slot[row] : -1;
            __nv_bfloat16* dst = nullptr;           // where this row's head goes (null: nowhere)
            if (row < M) {
                if (is_q) dst = reinterpret_cast<__nv_bfloat16*>(out) + ((size_t)row * ex.nh + head) * BN;
                else if (sl >= 0) {
                    const int kvh = is_k ? head - ex.nh : head - ex.nh - ex.nkv;
                    dst = ex.cache + (size_t)(sl / ex.page_size) * 2 * ex.nkv * ex.page_size * BN + (is_k ? 0 : (size_t)ex.nkv * ex.page_size * BN) +
                          ((size_t)kvh * ex.page_size + sl % ex.page_size) * BN;
                }
            }
#pragma unroll
            for (int c = 0; c < HALF; c += 32) {
                uint32_t ar[32], br[32];            // columns c .. c+31 and their partners HALF + c ..
                __syncwarp();
                tmem_ld32(lane_base + c, ar);
                tmem_ld32(lane_base + HALF + c, br);
                if (dst) {
                    uint32_t pa[16], pb[16];
#pragma unroll
                    for (int j = 0; j < 32; j += 2) {
                        float ra[2], rb[2];
#pragma unroll
                        for (int e = 0; e < 2; e++) {
                            const float a = __bfloat162float(__float2bfloat16_rn(__uint_as_float(ar[j + e])));
                            const float b = __bfloat162float(__float2bfloat16_rn(__uint_as_float(br[j + e])));
                            if (is_q || is_k) {
                                const int ti = c + j + e;                  // index into this row of the tables
                                const float4 c4 = rc[ti / 4], s4 = rs[ti / 4];
                                const float cs = (ti & 3) == 0 ? c4.x : (ti & 3) == 1 ? c4.y : (ti & 3) == 2 ? c4.z : c4.w;
                                const float sn = (ti & 3) == 0 ? s4.x : (ti & 3) == 1 ? s4.y : (ti & 3) == 2 ? s4.z : s4.w;
                                ra[e] = a * cs - b * sn;
                                rb[e] = b * cs + a * sn;
                            } else { ra[e] = a; rb[e] = b; }
                        }
                        __nv_bfloat162 va = __floats2bfloat162_rn(ra[0], ra[1]), vb = __floats2bfloat162_rn(rb[0], rb[1]);
                        pa[j / 2] = *reinterpret_cast<uint32_t*>(&va);
                        pb[j / 2] = *reinterpret_cast<uint32_t*>(&vb);
                    }
#pragma unroll
                    for (int j = 0; j < 4; j++) {
                        *reinterpret_cast<uint4*>(dst + c + 8 * j) = make_uint4(pa[4 * j], pa[4 * j + 1], pa[4 * j + 2], pa[4 * j + 3]);
                        *reinterpret_cast<uint4*>(dst + HALF + c + 8 * j) = make_uint4(pb[4 * j], pb[4 * j + 1], pb[4 * j + 2], pb[4 * j + 3]);
                    }
                }
            }
        } else if (EPI == TC_ACC && ex.tma_out) {
            // The residual sum by TMA: the tile goes into shared memory (the stages are free: every product has read them)
            // as boxes of 128 rows x 32 columns in the 128-byte swizzle, and one lane adds each box into out with a bulk
            // reduction, which clips rows and columns beyond the matrix.  A thread that wrote its own row's 32 columns
            // with 16-byte stores touched 32 different lines an instruction, and the old values had to be read the same
            // way: measured inside a 2,048-token prompt the epilogue was 2.2 of a tile's 9.4 microseconds.
            tc_fence_after();
            const int r_loc = quarter * 32 + lane;
#pragma unroll
            for (int c = 0; c < BN; c += 32) {
                uint32_t r[32];
                __syncwarp();
                tmem_ld32(tmem_base + ((uint32_t)(quarter * 32) << 16) + c, r);
                uint8_t* box = smem + (c / 32) * (TC_BM * 128) + r_loc * 128;
#pragma unroll
                for (int j = 0; j < 8; j++)
                    *reinterpret_cast<uint4*>(box + ((j ^ (r_loc & 7)) << 4)) = make_uint4(r[4 * j], r[4 * j + 1], r[4 * j + 2], r[4 * j + 3]);
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            asm volatile("bar.sync 1, 128;" ::: "memory");              // the four epilogue warps
            if (warp == 2 && lane == 0) {
#pragma unroll
                for (int c = 0; c < BN; c += 32) {
                    if (n0 + c < N)
                        asm volatile("cp.reduce.async.bulk.tensor.2d.global.shared::cta.add.tile.bulk_group [%0, {%2, %3}], [%1];"
                                     ::"l"(&map_out), "r"(smem_u32(smem + (c / 32) * (TC_BM * 128))), "r"(n0 + c), "r"(m0) : "memory");
                }
                asm volatile("cp.async.bulk.commit_group;" ::: "memory");
                asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
            }
        } else {
            tc_fence_after();
#pragma unroll
            for (int c = 0; c < BN; c += 32) {
                uint32_t r[32];
                __syncwarp();
                tmem_ld32(tmem_base + ((uint32_t)(quarter * 32) << 16) + c, r);
                const int col = n0 + c;
                const bool whole = col + 32 <= N;
                if (row >= M || col >= N) {
                    // nothing of this thread's to store
                } else if (EPI == TC_SAME) {
                    __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(out) + (size_t)row * N + col;
                    if (whole && (N % 8 == 0)) {
#pragma unroll
                        for (int j = 0; j < 32; j += 8) {
                            uint4 v;
                            __nv_bfloat162 p0 = __floats2bfloat162_rn(__uint_as_float(r[j]), __uint_as_float(r[j + 1]));
                            __nv_bfloat162 p1 = __floats2bfloat162_rn(__uint_as_float(r[j + 2]), __uint_as_float(r[j + 3]));
                            __nv_bfloat162 p2 = __floats2bfloat162_rn(__uint_as_float(r[j + 4]), __uint_as_float(r[j + 5]));
                            __nv_bfloat162 p3 = __floats2bfloat162_rn(__uint_as_float(r[j + 6]), __uint_as_float(r[j + 7]));
                            v.x = *reinterpret_cast<uint32_t*>(&p0); v.y = *reinterpret_cast<uint32_t*>(&p1);
                            v.z = *reinterpret_cast<uint32_t*>(&p2); v.w = *reinterpret_cast<uint32_t*>(&p3);
                            *reinterpret_cast<uint4*>(o + j) = v;
                        }
                    } else {
                        for (int j = 0; j < 32 && col + j < N; j++) o[j] = __float2bfloat16_rn(__uint_as_float(r[j]));
                    }
                } else {
                    float* o = reinterpret_cast<float*>(out) + (size_t)row * N + col;
                    if (whole && (N % 4 == 0)) {
                        float4 prev[8];
                        if (EPI == TC_ACC) {
                            if (c < 64) {                  // read before the wait
#pragma unroll
                                for (int j = 0; j < 8; j++) prev[j] = pre[c / 32][j];
                            } else {                       // all eight reads are issued before any is used
#pragma unroll
                                for (int j = 0; j < 8; j++) prev[j] = *reinterpret_cast<const float4*>(o + 4 * j);
                            }
                        }
#pragma unroll
                        for (int j = 0; j < 8; j++) {
                            float4 v = make_float4(__uint_as_float(r[4 * j]), __uint_as_float(r[4 * j + 1]), __uint_as_float(r[4 * j + 2]),
                                                   __uint_as_float(r[4 * j + 3]));
                            if (EPI == TC_ACC) { v.x += prev[j].x; v.y += prev[j].y; v.z += prev[j].z; v.w += prev[j].w; }
                            *reinterpret_cast<float4*>(o + 4 * j) = v;
                        }
                    } else {
                        for (int j = 0; j < 32 && col + j < N; j++) {
                            if (EPI == TC_ACC) o[j] += __uint_as_float(r[j]);
                            else o[j] = __uint_as_float(r[j]);
                        }
                    }
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        if (failed) __nanosleep(200000);      // after a failed wait: let copies in flight land
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(BN) : "memory");
    }
}

// ---------------------------------------------------------------------------------------------------------------
// The wide variant for large products: a block (one a multiprocessor, as many blocks as multiprocessors) walks over
// output tiles of 128 x 256, and two accumulators in tensor memory (2 x 256 columns, all there is) let the eight
// epilogue warps drain one tile while the tensor core fills the next.  A 128 x 256 tile reads a quarter fewer bytes
// a flop from the second-level cache than 128 x 128 (which that traffic bounded at about 60 % of the tensor peak),
// and N = 256 instructions take the tensor core longer than they take their thread to issue.
// SwiGLU: a tile is 128 gate rows and the 128 up rows of the same columns.  BNW, the tile's width in weight rows, is a
// parameter of the kernel: 256, or 192 (96 gate and 96 up rows) where the launcher finds that a block's last round of
// the wider tile would be mostly empty.
constexpr int TW_BN = 256, TW_STAGES = 4, TW_THREADS = 320;      // warps 0 and 1 feed and issue; eight warps drain the accumulators

template <int EPI, int HD = 0, int BNW = TW_BN>
__global__ void __launch_bounds__(TW_THREADS, 1) linear_tcgen05_wide_kernel(const __grid_constant__ CUtensorMap map_x,
                                                                         const __grid_constant__ CUtensorMap map_w,
                                                                         const __grid_constant__ CUtensorMap map_out, void* __restrict__ out,
                                                                         int M, int N, int K, const WaitCtl wc, const TcExtra ex) {
    constexpr uint32_t A_BYTES = TC_BM * TC_BK * 2, B_BYTES = BNW * TC_BK * 2, STAGE_BYTES = A_BYTES + B_BYTES;
    constexpr uint32_t TM_COLS = 2 * BNW <= 256 ? 256 : 512;      // the two accumulators; tensor memory comes in powers of two
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + TW_STAGES * STAGE_BYTES);
    uint64_t* empty = full + TW_STAGES;
    uint64_t* acc_full = empty + TW_STAGES;       // [2]
    uint64_t* acc_empty = acc_full + 2;           // [2]
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
    __shared__ int failed;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int num_kb = (K + TC_BK - 1) / TC_BK;
    const int tile_cols = EPI == TC_SWIGLU ? BNW / 2 : BNW;                // output columns of a tile
    const int out_cols = EPI == TC_SWIGLU ? ex.inter : N;
    const int tiles_m = (M + TC_BM - 1) / TC_BM, tiles_n = (out_cols + tile_cols - 1) / tile_cols;
    const int num_tiles = tiles_m * tiles_n;      // tile t: rows (t % tiles_m) * 128, columns (t / tiles_m) * tile_cols

    if (threadIdx.x == 0) {
        failed = 0;
        for (int s = 0; s < TW_STAGES; s++) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
        for (int b = 0; b < 2; b++) { mbar_init(&acc_full[b], 1); mbar_init(&acc_empty[b], 8); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(TM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        if (lane == 0) {
            int kc = 0;                            // stages filled so far, over all of this block's tiles
            bool ok = true;
            for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
                const int m0 = (t % tiles_m) * TC_BM, n0 = (t / tiles_m) * tile_cols;
                for (int kb = 0; kb < num_kb; kb++, kc++) {
                    const int s = kc % TW_STAGES;
                    if (kc >= TW_STAGES && !mbar_wait(&empty[s], ((kc / TW_STAGES) - 1) & 1, wc.cycles)) { give_up(wc.error, &failed, 31); ok = false; break; }
                    if (kc == wc.skip_stage) continue;      // left unarmed and unfilled: a test of the give-up path
                    mbar_expect_tx(&full[s], STAGE_BYTES);
                    tma_load_2d(smem + s * STAGE_BYTES, &map_x, kb * TC_BK, m0, &full[s]);
                    if (EPI == TC_SWIGLU) {        // the map's box is 128 rows: gate rows, then the same rows of up
                        tma_load_2d(smem + s * STAGE_BYTES + A_BYTES, &map_w, kb * TC_BK, n0, &full[s]);
                        tma_load_2d(smem + s * STAGE_BYTES + A_BYTES + B_BYTES / 2, &map_w, kb * TC_BK, ex.inter + n0, &full[s]);
                    } else {
                        tma_load_2d(smem + s * STAGE_BYTES + A_BYTES, &map_w, kb * TC_BK, n0, &full[s]);
                    }
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            const uint32_t idesc = umma_idesc_bf16(TC_BM, BNW);
            const uint32_t a_lo0 = umma_desc_lo(smem_u32(smem));      // low words of the descriptors (see umma_bf16_lo)
            int kc = 0, j = 0;
            bool ok = true;
            for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x, j++) {
                const int b = j & 1;
                if (j >= 2 && !mbar_wait(&acc_empty[b], ((j >> 1) - 1) & 1, wc.cycles)) { give_up(wc.error, &failed, 32); break; }
                tc_fence_after();
                for (int kb = 0; kb < num_kb; kb++, kc++) {
                    const int s = kc % TW_STAGES;
                    if (!mbar_wait(&full[s], (kc / TW_STAGES) & 1, wc.cycles)) { give_up(wc.error, &failed, 33); ok = false; break; }
                    tc_fence_after();
                    const uint32_t a_lo = a_lo0 + s * (STAGE_BYTES >> 4), b_lo = a_lo + (A_BYTES >> 4);
#pragma unroll
                    for (int k = 0; k < TC_BK / 16; k++) umma_bf16_lo(tmem_base + b * BNW, a_lo + 2 * k, b_lo + 2 * k, idesc, (kb | k) != 0);
                    umma_commit(&empty[s]);
                }
                if (ok) umma_commit(&acc_full[b]);
            }
        }
    } else {
        // epilogue: warp w reads lanes 32*(w%4) .. +31 of the accumulator (the lanes a warp may read), one output row per
        // thread; the two warps of a lane quarter take half of the tile's columns each
        const int quarter = warp & 3, half = (warp - 2) >> 2;
        const uint32_t lane_base = tmem_base + ((uint32_t)(quarter * 32) << 16);
        int j = 0;
        bool ok = true;
        for (int t = blockIdx.x; t < num_tiles; t += gridDim.x, j++) {
            const int b = j & 1;
            const int row = (t % tiles_m) * TC_BM + quarter * 32 + lane, n0 = (t / tiles_m) * tile_cols;
            if (ok && !__all_sync(0xffffffffu, mbar_wait(&acc_full[b], (j >> 1) & 1, wc.cycles))) { if (lane == 0) give_up(wc.error, &failed, 34); ok = false; }
            // The block's last tile of a residual sum goes out by TMA reductions from shared memory (see the narrow kernel): its
            // epilogue hides behind no further tile, and every stage is free by now.  The eight epilogue warps meet for it,
            // so they go on together or not at all.
            const bool by_tma = EPI == TC_ACC && ex.tma_out && t + (int)gridDim.x >= num_tiles;
            if (by_tma) {
                asm volatile("bar.sync 2, 256;" ::: "memory");
                if (*reinterpret_cast<volatile int*>(&failed)) ok = false;
            }
            if (ok && by_tma) {
                tc_fence_after();
                const uint32_t acc = lane_base + b * BNW;
                const int r_loc = quarter * 32 + lane;
#pragma unroll 1
                for (int c = half * (BNW / 2); c < (half + 1) * (BNW / 2); c += 32) {
                    uint32_t r[32];
                    tmem_ld32(acc + c, r);
                    tmem_loaded(r);
                    uint8_t* box = smem + (c / 32) * (TC_BM * 128) + r_loc * 128;
#pragma unroll
                    for (int q = 0; q < 8; q++)
                        *reinterpret_cast<uint4*>(box + ((q ^ (r_loc & 7)) << 4)) = make_uint4(r[4 * q], r[4 * q + 1], r[4 * q + 2], r[4 * q + 3]);
                }
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                tc_fence_before();
                asm volatile("bar.sync 2, 256;" ::: "memory");
                if (warp == 2 && lane == 0) {
                    const int m0 = (t % tiles_m) * TC_BM;
                    for (int c = 0; c < BNW; c += 32) {
                        if (n0 + c < N)
                            asm volatile("cp.reduce.async.bulk.tensor.2d.global.shared::cta.add.tile.bulk_group [%0, {%2, %3}], [%1];"
                                         ::"l"(&map_out), "r"(smem_u32(smem + (c / 32) * (TC_BM * 128))), "r"(n0 + c), "r"(m0) : "memory");
                    }
                    asm volatile("cp.async.bulk.commit_group;" ::: "memory");
                    asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
                }
            } else if (ok) {
                tc_fence_after();
                const uint32_t acc = lane_base + b * BNW;
                if (EPI == TC_SWIGLU) {
#pragma unroll 1
                    // the tile's gate columns in chunks of 32: the first of a lane quarter's two warps takes the first half of
                    // them (rounded up), the second the rest
                    constexpr int CHUNKS = BNW / 2 / 32, SPLIT = (CHUNKS + 1) / 2;
                    for (int c = (half == 0 ? 0 : SPLIT) * 32; c < (half == 0 ? SPLIT : CHUNKS) * 32; c += 32) {
                        uint32_t gr[32], ur[32];
                        tmem_ld32_nowait(acc + c, gr);
                        tmem_ld32_nowait(acc + BNW / 2 + c, ur);
                        tmem_wait_ld();
                        tmem_loaded(gr);
                        tmem_loaded(ur);
                        const int col = n0 + c;
                        if (row < M && col < ex.inter) {
                            __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(out) + (size_t)row * ex.inter + col;
                            uint32_t packed[16];
#pragma unroll
                            for (int q = 0; q < 32; q += 2) {
                                float v[2];
#pragma unroll
                                for (int e = 0; e < 2; e++) {
                                    const float gte = __bfloat162float(__float2bfloat16_rn(__uint_as_float(gr[q + e])));
                                    const float up = __bfloat162float(__float2bfloat16_rn(__uint_as_float(ur[q + e])));
                                    v[e] = tc_silu_mul(gte, up);
                                }
                                __nv_bfloat162 pk = __floats2bfloat162_rn(v[0], v[1]);
                                packed[q / 2] = *reinterpret_cast<uint32_t*>(&pk);
                            }
                            if (col + 32 <= ex.inter && (ex.inter % 8 == 0)) {
#pragma unroll
                                for (int q = 0; q < 4; q++)
                                    *reinterpret_cast<uint4*>(o + 8 * q) = make_uint4(packed[4 * q], packed[4 * q + 1], packed[4 * q + 2], packed[4 * q + 3]);
                            } else {
                                for (int q = 0; q < 32 && col + q < ex.inter; q++)
                                    o[q] = __ushort_as_bfloat16((unsigned short)((packed[q / 2] >> ((q & 1) * 16)) & 0xffffu));
                            }
                        }
                    }
                } else if (EPI == TC_ROPE) {
                    // the tile is 256 / HD heads: q heads, then k heads, then v heads (see the narrow kernel)
                    constexpr int HDX = HD > 0 ? HD : 64, HALF = HDX / 2;
                    const int sl = row < M ? ex.slot[row] : -1;
                    const int p0 = row < M ? ex.positions[row] : 0;
#pragma unroll 1
                    for (int hh = half * (BNW / HDX / 2); hh < (half + 1) * (BNW / HDX / 2); hh++) {
                        const int head = n0 / HDX + hh;
                        if (head >= ex.nh + 2 * ex.nkv) break;          // the same for the whole warp
                        const bool is_q = head < ex.nh, is_k = !is_q && head < ex.nh + ex.nkv;
                        __nv_bfloat16* dst = nullptr;                   // where this row's head goes (null: nowhere)
                        if (row < M) {
                            if (is_q) dst = reinterpret_cast<__nv_bfloat16*>(out) + ((size_t)row * ex.nh + head) * HDX;
                            else if (sl >= 0) {
                                const int kvh = is_k ? head - ex.nh : head - ex.nh - ex.nkv;
                                dst = ex.cache + (size_t)(sl / ex.page_size) * 2 * ex.nkv * ex.page_size * HDX +
                                      (is_k ? 0 : (size_t)ex.nkv * ex.page_size * HDX) + ((size_t)kvh * ex.page_size + sl % ex.page_size) * HDX;
                            }
                        }
#pragma unroll 1
                        for (int c = 0; c < HALF; c += 32) {
                            uint32_t ar[32], br[32];                    // columns c .. c+31 of the head and their partners HALF + c ..
                            tmem_ld32_nowait(acc + hh * HDX + c, ar);
                            tmem_ld32_nowait(acc + hh * HDX + HALF + c, br);
                            tmem_wait_ld();
                            tmem_loaded(ar);
                            tmem_loaded(br);
                            if (!dst) continue;
                            const float4* cp = reinterpret_cast<const float4*>(ex.cos_t + (size_t)p0 * HALF + c);
                            const float4* sp = reinterpret_cast<const float4*>(ex.sin_t + (size_t)p0 * HALF + c);
                            uint32_t pa[16], pb[16];
#pragma unroll
                            for (int q = 0; q < 32; q += 4) {
                                float4 c4 = make_float4(1.0f, 1.0f, 1.0f, 1.0f), s4 = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
                                if (is_q || is_k) { c4 = cp[q / 4]; s4 = sp[q / 4]; }
                                const float cs[4] = {c4.x, c4.y, c4.z, c4.w}, sn[4] = {s4.x, s4.y, s4.z, s4.w};
                                float ra[4], rb[4];
#pragma unroll
                                for (int e = 0; e < 4; e++) {
                                    const float a = __bfloat162float(__float2bfloat16_rn(__uint_as_float(ar[q + e])));
                                    const float b2 = __bfloat162float(__float2bfloat16_rn(__uint_as_float(br[q + e])));
                                    ra[e] = a * cs[e] - b2 * sn[e];
                                    rb[e] = b2 * cs[e] + a * sn[e];
                                }
                                __nv_bfloat162 va0 = __floats2bfloat162_rn(ra[0], ra[1]), va1 = __floats2bfloat162_rn(ra[2], ra[3]);
                                __nv_bfloat162 vb0 = __floats2bfloat162_rn(rb[0], rb[1]), vb1 = __floats2bfloat162_rn(rb[2], rb[3]);
                                pa[q / 2] = *reinterpret_cast<uint32_t*>(&va0); pa[q / 2 + 1] = *reinterpret_cast<uint32_t*>(&va1);
                                pb[q / 2] = *reinterpret_cast<uint32_t*>(&vb0); pb[q / 2 + 1] = *reinterpret_cast<uint32_t*>(&vb1);
                            }
#pragma unroll
                            for (int q = 0; q < 4; q++) {
                                *reinterpret_cast<uint4*>(dst + c + 8 * q) = make_uint4(pa[4 * q], pa[4 * q + 1], pa[4 * q + 2], pa[4 * q + 3]);
                                *reinterpret_cast<uint4*>(dst + HALF + c + 8 * q) = make_uint4(pb[4 * q], pb[4 * q + 1], pb[4 * q + 2], pb[4 * q + 3]);
                            }
                        }
                    }
                } else {
#pragma unroll 1
                    for (int c = half * (BNW / 2); c < (half + 1) * (BNW / 2); c += 32) {
                        uint32_t r[32];
                        tmem_ld32(acc + c, r);
                        tmem_loaded(r);
                        const int col = n0 + c;
                        if (row >= M || col >= N) continue;
                        const bool whole = col + 32 <= N;
                        if (EPI == TC_SAME) {
                            __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(out) + (size_t)row * N + col;
                            if (whole && (N % 8 == 0)) {
#pragma unroll
                                for (int q = 0; q < 32; q += 8) {
                                    uint4 v;
                                    __nv_bfloat162 p0 = __floats2bfloat162_rn(__uint_as_float(r[q]), __uint_as_float(r[q + 1]));
                                    __nv_bfloat162 p1 = __floats2bfloat162_rn(__uint_as_float(r[q + 2]), __uint_as_float(r[q + 3]));
                                    __nv_bfloat162 p2 = __floats2bfloat162_rn(__uint_as_float(r[q + 4]), __uint_as_float(r[q + 5]));
                                    __nv_bfloat162 p3 = __floats2bfloat162_rn(__uint_as_float(r[q + 6]), __uint_as_float(r[q + 7]));
                                    v.x = *reinterpret_cast<uint32_t*>(&p0); v.y = *reinterpret_cast<uint32_t*>(&p1);
                                    v.z = *reinterpret_cast<uint32_t*>(&p2); v.w = *reinterpret_cast<uint32_t*>(&p3);
                                    *reinterpret_cast<uint4*>(o + q) = v;
                                }
                            } else {
                                for (int q = 0; q < 32 && col + q < N; q++) o[q] = __float2bfloat16_rn(__uint_as_float(r[q]));
                            }
                        } else {
                            float* o = reinterpret_cast<float*>(out) + (size_t)row * N + col;
                            if (whole && (N % 4 == 0)) {
                                float4 prev[8];
                                if (EPI == TC_ACC) {           // all eight reads are issued before any is used
#pragma unroll
                                    for (int q = 0; q < 8; q++) prev[q] = *reinterpret_cast<const float4*>(o + 4 * q);
                                }
#pragma unroll
                                for (int q = 0; q < 8; q++) {
                                    float4 v = make_float4(__uint_as_float(r[4 * q]), __uint_as_float(r[4 * q + 1]), __uint_as_float(r[4 * q + 2]),
                                                           __uint_as_float(r[4 * q + 3]));
                                    if (EPI == TC_ACC) { v.x += prev[q].x; v.y += prev[q].y; v.z += prev[q].z; v.w += prev[q].w; }
                                    *reinterpret_cast<float4*>(o + 4 * q) = v;
                                }
                            } else {
                                for (int q = 0; q < 32 && col + q < N; q++) {
                                    if (EPI == TC_ACC) o[q] += __uint_as_float(r[q]);
                                    else o[q] = __uint_as_float(r[q]);
                                }
                            }
                        }
                    }
                }
                tc_fence_before();
            }
            __syncwarp();
            if (lane == 0) mbar_arrive_plain(&acc_empty[b]);      // kept even after a failed wait: nobody waits for this warp without a limit
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        if (failed) __nanosleep(200000);      // after a failed wait: let copies in flight land
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TM_COLS) : "memory");
    }
}

// A [rows, cols] bfloat16 matrix with row stride ld (elements), read in boxes of box_rows x 64 columns.
static bool make_map(CUtensorMap* map, const void* base, int rows, int cols, int ld, int box_rows) {
    EncodeTiledFn enc = encode_tiled();
    if (!enc) return false;
    cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
    cuuint32_t box[2] = {(cuuint32_t)TC_BK, (cuuint32_t)box_rows};
    cuuint32_t elem[2] = {1, 1};
    return enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE,
               CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// out [rows, cols] float32, dense: added into in boxes of 128 rows x 32 columns, 128-byte swizzle.
static bool make_out_map(CUtensorMap* map, void* base, int rows, int cols) {
    EncodeTiledFn enc = encode_tiled();
    if (!enc) return false;
    cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)cols * 4};
    cuuint32_t box[2] = {32u, (cuuint32_t)TC_BM};
    cuuint32_t elem[2] = {1, 1};
    return enc(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, base, dims, strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE,
               CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <int BN, int EPI>
static int launch_tc(const CUtensorMap& mx, const CUtensorMap& mw, void* out, int M, int N, int K, int* error, cudaStream_t stream,
                     const TcExtra& ex = TcExtra{}) {
    const WaitCtl wc = wait_ctl(error, WAIT_FAMILY_LINEAR);
    const size_t smem = (size_t)TcStages<BN>::N * (TC_BM * TC_BK * 2 + BN * TC_BK * 2) + 1024 + 128;
    TcExtra exx = ex;
    CUtensorMap mo = mx;                               // (a valid map for the epilogues that do not use it)
    exx.tma_out = 0;
    if (EPI == TC_ACC && N % 4 == 0 && ((uintptr_t)out % 16 == 0) && make_out_map(&mo, out, M, N)) exx.tma_out = 1;
    auto kern = linear_tcgen05_kernel<BN, EPI>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    const int tile_cols = EPI == TC_SWIGLU ? BN / 2 : BN;
    const int cols = EPI == TC_SWIGLU ? ex.inter : N;
    dim3 grid((cols + tile_cols - 1) / tile_cols, (M + TC_BM - 1) / TC_BM);
    return launch_dependent(kern, grid, dim3(TC_THREADS), smem, stream, mx, mw, mo, out, M, N, K, wc, exx);
}

static int sm_count() {
    static int n = 0;
    if (!n) {
        int dev = 0;
        cudaGetDevice(&dev);
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    }
    return n;
}

// Whether the wide variant takes a product.  Measured at M = 2,048 (bench.py --only-gemm, replayed from a graph): it wins
// where a block gets more than one tile (the epilogue of one hides behind the main loop of the next; with eight epilogue
// warps also at K = 576, where a tile's main loop is only nine stages long) or where K is long enough that the main loop
// is nearly all of a tile's time; with one short tile a block the narrow kernel's two blocks a multiprocessor do better.
// tile_cols: output columns of a wide tile.  VITNA_TCGEN05_WIDE=0 or 1 overrides (for measurements).
static bool wide_takes(int M, int out_cols, int K, int tile_cols = TW_BN) {
    static int forced = -1;
    if (forced < 0) {
        const char* e = getenv("VITNA_TCGEN05_WIDE");
        forced = e ? (e[0] == '1' ? 1 : 0) : 2;
    }
    if (forced != 2) return forced == 1;
    if (M < 512 || out_cols < 1024 || K < 512) return false;
    const long long tiles = (long long)((M + TC_BM - 1) / TC_BM) * ((out_cols + tile_cols - 1) / tile_cols);
    return K >= 2048 || tiles * 4 >= (long long)sm_count() * 5;
}

template <int EPI, int HD = 0, int BNW = TW_BN>
static int launch_wide(const CUtensorMap& mx, const CUtensorMap& mw, void* out, int M, int N, int K, int* error, cudaStream_t stream,
                       const TcExtra& ex = TcExtra{}) {
    const WaitCtl wc = wait_ctl(error, WAIT_FAMILY_LINEAR_WIDE);
    const size_t smem = (size_t)TW_STAGES * (TC_BM * TC_BK * 2 + BNW * TC_BK * 2) + 1024 + 128;
    TcExtra exx = ex;
    CUtensorMap mo = mx;                               // (a valid map for the epilogues that do not use it)
    exx.tma_out = 0;
    if (EPI == TC_ACC && N % 4 == 0 && ((uintptr_t)out % 16 == 0) && make_out_map(&mo, out, M, N)) exx.tma_out = 1;
    auto kern = linear_tcgen05_wide_kernel<EPI, HD, BNW>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    const int tile_cols = EPI == TC_SWIGLU ? BNW / 2 : BNW;
    const int cols = EPI == TC_SWIGLU ? ex.inter : N;
    const long long tiles = (long long)((M + TC_BM - 1) / TC_BM) * ((cols + tile_cols - 1) / tile_cols);
    const int grid = tiles < sm_count() ? (int)tiles : sm_count();
    return launch_plain(kern, dim3(grid), dim3(TW_THREADS), smem, stream, mx, mw, mo, out, M, N, K, wc, exx);
}

}  // namespace vk

using namespace vk;

// x [M, K] bfloat16 with row stride ldx, w [N, K] bfloat16, out [M, N]: mode 0 bfloat16, 1 float32, 2 float32 +=.
// K and ldx multiples of 8, pointers 16-byte aligned.  error: a word the kernel sets (non-zero) if a bounded wait ran out.
VK_API int vk_linear_tcgen05(const void* x, const void* w, void* out, int M, int N, int K, int ldx, int mode, int* error,
                             cudaStream_t stream) {
    if (M <= 0 || N <= 0) return VK_OK;
    if (K <= 0 || ldx < K || mode < 0 || mode > 2 || !error) return VK_BAD_SHAPE;
    if (K % 8 != 0 || ldx % 8 != 0) return VK_BAD_SHAPE;
    if (((uintptr_t)x % 16) || ((uintptr_t)w % 16) || ((uintptr_t)out % 16)) return VK_BAD_ALIGNMENT;
    const int bn = N >= 2048 ? 128 : 64;
    if ((M + TC_BM - 1) / TC_BM > 65535) return VK_TOO_LARGE;
    if (wide_takes(M, N, K)) {
        CUtensorMap wx, ww;
        if (!make_map(&wx, x, M, K, ldx, TC_BM) || !make_map(&ww, w, N, K, K, TW_BN)) return VK_BAD_SHAPE;
        if (mode == 0) return launch_wide<TC_SAME>(wx, ww, out, M, N, K, error, stream);
        if (mode == 1) return launch_wide<TC_F32>(wx, ww, out, M, N, K, error, stream);
        return launch_wide<TC_ACC>(wx, ww, out, M, N, K, error, stream);
    }
    CUtensorMap mx, mw;
    if (!make_map(&mx, x, M, K, ldx, TC_BM) || !make_map(&mw, w, N, K, K, bn)) return VK_BAD_SHAPE;
#define GO(BN, EPI) return launch_tc<BN, EPI>(mx, mw, out, M, N, K, error, stream)
    if (bn == 128) {
        if (mode == 0) GO(128, TC_SAME);
        if (mode == 1) GO(128, TC_F32);
        GO(128, TC_ACC);
    }
    if (mode == 0) GO(64, TC_SAME);
    if (mode == 1) GO(64, TC_F32);
    GO(64, TC_ACC);
#undef GO
}

// x [M, K] bfloat16 (row stride ldx), w [2*inter, K] bfloat16 with gate rows then up rows, out [M, inter] bfloat16 =
// silu(x gate^T) * (x up^T).  inter a multiple of 8.
VK_API int vk_linear_tcgen05_swiglu(const void* x, const void* w, void* out, int M, int inter, int K, int ldx, int* error,
                                    cudaStream_t stream) {
    if (M <= 0 || inter <= 0) return VK_OK;
    if (K <= 0 || ldx < K || !error || K % 8 != 0 || ldx % 8 != 0 || inter % 8 != 0) return VK_BAD_SHAPE;
    if (((uintptr_t)x % 16) || ((uintptr_t)w % 16) || ((uintptr_t)out % 16)) return VK_BAD_ALIGNMENT;
    if ((M + TC_BM - 1) / TC_BM > 65535) return VK_TOO_LARGE;
    CUtensorMap mx, mw;
    TcExtra ex{};
    ex.inter = inter;
    if (wide_takes(M, inter, K, TW_BN / 2)) {
        // Tiles of 128 x 96 output columns (192 weight rows) where they come out sooner than tiles of 128 x 128: a block
        // walks through ceil(tiles / blocks) tiles, and at the 135M and 360M sizes the last round of the wider tile is
        // mostly empty (192 tiles on 148 multiprocessors: two rounds of 256 columns against two of 192).
        const long long tiles_m = (M + TC_BM - 1) / TC_BM, sms = sm_count();
        const long long rounds256 = (tiles_m * ((inter + 127) / 128) + sms - 1) / sms, rounds192 = (tiles_m * ((inter + 95) / 96) + sms - 1) / sms;
        if (rounds192 * 192 < rounds256 * 256) {
            if (!make_map(&mx, x, M, K, ldx, TC_BM) || !make_map(&mw, w, 2 * inter, K, K, 96)) return VK_BAD_SHAPE;
            return launch_wide<TC_SWIGLU, 0, 192>(mx, mw, out, M, 2 * inter, K, error, stream, ex);
        }
        if (!make_map(&mx, x, M, K, ldx, TC_BM) || !make_map(&mw, w, 2 * inter, K, K, TW_BN / 2)) return VK_BAD_SHAPE;
        return launch_wide<TC_SWIGLU>(mx, mw, out, M, 2 * inter, K, error, stream, ex);
    }
    if (!make_map(&mx, x, M, K, ldx, TC_BM) || !make_map(&mw, w, 2 * inter, K, K, 64)) return VK_BAD_SHAPE;
    return launch_tc<128, TC_SWIGLU>(mx, mw, out, M, 2 * inter, K, error, stream, ex);
}

// x [M, K] bfloat16, w [(nh + 2*nkv) * hd, K] bfloat16 (q heads, k heads, v heads); q_out [M, nh*hd] bfloat16 gets the
// rotated q, the layer's cache ([pages][2][nkv][page_size][hd]) gets rotated k and v at slot[m] (-1: no write).
// hd 64 or 128; cos, sin [positions, hd/2] float32.
VK_API int vk_linear_tcgen05_rope(const void* x, const void* w, void* q_out, int M, int K, int ldx, const int32_t* positions,
                                  const float* cos_t, const float* sin_t, const int32_t* slot, void* cache, int nh, int nkv, int hd,
                                  int page_size, int* error, cudaStream_t stream) {
    if (M <= 0) return VK_OK;
    if (K <= 0 || ldx < K || !error || K % 8 != 0 || ldx % 8 != 0 || nh <= 0 || nkv <= 0 || page_size <= 0 || !positions || !cos_t ||
        !sin_t || !slot || !cache)
        return VK_BAD_SHAPE;
    if (hd != 64 && hd != 128) return VK_BAD_SHAPE;
    if (((uintptr_t)x % 16) || ((uintptr_t)w % 16) || ((uintptr_t)q_out % 16) || ((uintptr_t)cache % 16)) return VK_BAD_ALIGNMENT;
    if ((M + TC_BM - 1) / TC_BM > 65535) return VK_TOO_LARGE;
    const int N = (nh + 2 * nkv) * hd;
    CUtensorMap mx, mw;
    if (!make_map(&mx, x, M, K, ldx, TC_BM) || !make_map(&mw, w, N, K, K, hd)) return VK_BAD_SHAPE;
    TcExtra ex{};
    ex.positions = positions; ex.cos_t = cos_t; ex.sin_t = sin_t; ex.slot = slot; ex.cache = (__nv_bfloat16*)cache;
    ex.nh = nh; ex.nkv = nkv; ex.hd = hd; ex.page_size = page_size;
    if (wide_takes(M, N, K)) {
        if (!make_map(&mw, w, N, K, K, TW_BN)) return VK_BAD_SHAPE;
        if (hd == 64) return launch_wide<TC_ROPE, 64>(mx, mw, q_out, M, N, K, error, stream, ex);
        return launch_wide<TC_ROPE, 128>(mx, mw, q_out, M, N, K, error, stream, ex);
    }
    if (hd == 64) return launch_tc<64, TC_ROPE>(mx, mw, q_out, M, N, K, error, stream, ex);
    return launch_tc<128, TC_ROPE>(mx, mw, q_out, M, N, K, error, stream, ex);
}
