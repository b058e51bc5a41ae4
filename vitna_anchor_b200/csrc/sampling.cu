// Choosing the next token on the device: greedy, or temperature with top-k
// and top-p, one block per row of logits.
//
// The rule is the reference's (engine/src/sampler.c:96-139): greedy takes the
// first of equal maxima; otherwise p_i = expf((l_i - max) / temperature),
// normalised by a sum in double; the ids are ordered by probability, larger
// first and the lower id first among equals; top-k keeps a prefix of that
// order, top-p the smallest prefix whose mass reaches top_p of what is kept
// (at least one token); one uniform u picks the first token whose cumulative
// mass in that order exceeds u * kept_mass.
//
// No sort is done.  The order is total, so "the first position of the order
// at which a running count or a running mass crosses a target" is found by
// descending the 32 bits of the key (~bits(p): ascending keys are descending
// probabilities) eight bits at a time with a histogram of counts and masses,
// and equal keys are resolved by id.  Masses are summed as 64-bit fixed-point
// integers (2^-62 units), so the sums are exact, and the same whatever the
// order the threads add in; the choice differs from a sequential
// double-precision walk only if u falls within about 1e-14 of a boundary.
//
// Scratch: probs [rows, vocab] float32, written and read by this kernel.
#include "common.cuh"

namespace vk {

constexpr int SAMPLE_THREADS = 1024;
constexpr double FIXED_ONE = 4611686018427387904.0;  // 2^62

struct Prefix {
    unsigned long long count;  // elements in the prefix
    unsigned long long mass;   // their mass, fixed point
    uint32_t key;              // key of the prefix's last element
    unsigned long long nth;    // which of the elements with that key (1-based, by id) is the last
};

__device__ __forceinline__ uint32_t key_of(float p) { return ~__float_as_uint(p); }
__device__ __forceinline__ unsigned long long fixed_of(float p) { return (unsigned long long)((double)p * FIXED_ONE); }

// mass_mode: 0 = no mass condition, 1 = stop when mass >= target, 2 = stop when mass > target.
// The prefix also stops when it holds `limit` elements.  Called by all threads of the block.
__device__ Prefix find_prefix(const float* __restrict__ probs, int n, int mass_mode, unsigned long long target,
                              unsigned long long limit, unsigned int* h_cnt, unsigned long long* h_mass, Prefix* result) {
    uint32_t prefix = 0;
    unsigned long long cnt_before = 0, mass_before = 0;
    for (int shift = 24; shift >= 0; shift -= 8) {
        for (int i = threadIdx.x; i < 256; i += blockDim.x) { h_cnt[i] = 0; h_mass[i] = 0; }
        __syncthreads();
        for (int i = threadIdx.x; i < n; i += blockDim.x) {
            const float p = probs[i];
            const uint32_t k = key_of(p);
            if (shift == 24 || (k >> (shift + 8)) == (prefix >> (shift + 8))) {
                const uint32_t d = (k >> shift) & 255u;
                atomicAdd(&h_cnt[d], 1u);
                atomicAdd(&h_mass[d], fixed_of(p));
            }
        }
        __syncthreads();
        if (threadIdx.x == 0) {
            unsigned long long c = cnt_before, m = mass_before;
            int chosen = -1, last_nonempty = -1;
            unsigned long long c_last = c, m_last = m;
            for (int b = 0; b < 256; b++) {
                if (h_cnt[b] == 0) continue;
                const unsigned long long ca = c + h_cnt[b], ma = m + h_mass[b];
                const bool hit = ca >= limit || (mass_mode == 1 && ma >= target) || (mass_mode == 2 && ma > target);
                last_nonempty = b; c_last = c; m_last = m;
                if (hit) { chosen = b; break; }
                c = ca; m = ma;
            }
            if (chosen < 0) { chosen = last_nonempty; c = c_last; m = m_last; }  // the target lies beyond the total: end at the last element
            result->count = c;
            result->mass = m;
            result->key = prefix | ((uint32_t)chosen << shift);
            result->nth = h_cnt[chosen];
        }
        __syncthreads();
        prefix = result->key;
        cnt_before = result->count;
        mass_before = result->mass;
        __syncthreads();
    }
    // All elements with key == prefix have the same probability; take as many as the conditions need.
    Prefix out;
    const unsigned long long ties = result->nth;
    const unsigned long long pm = fixed_of(__uint_as_float(~prefix));
    unsigned long long need = ties;
    if (mass_mode != 0 && pm > 0 && target >= mass_before) {
        const unsigned long long gap = target - mass_before;
        need = (mass_mode == 1) ? (gap + pm - 1) / pm : gap / pm + 1;
        if (need < 1) need = 1;
    } else if (mass_mode != 0 && target < mass_before) {
        need = 1;
    }
    if (need > ties) need = ties;
    if (limit > cnt_before && need > limit - cnt_before) need = limit - cnt_before;
    if (need < 1) need = 1;
    out.count = cnt_before + need;
    out.mass = mass_before + need * pm;
    out.key = prefix;
    out.nth = need;
    return out;
}

// The id of the nth (1-based) element, in id order, whose key equals `key`.
__device__ int find_nth_with_key(const float* __restrict__ probs, int n, uint32_t key, unsigned long long nth,
                                 unsigned int* counts, int* answer) {
    const int chunk = (n + blockDim.x - 1) / blockDim.x;
    const int lo = threadIdx.x * chunk, hi = min(n, lo + chunk);
    unsigned int c = 0;
    for (int i = lo; i < hi; i++) c += key_of(probs[i]) == key;
    counts[threadIdx.x] = c;
    __syncthreads();
    if (threadIdx.x == 0) {
        unsigned long long seen = 0;
        int owner = -1;
        for (int t = 0; t < (int)blockDim.x; t++) {
            if (seen + counts[t] >= nth) { owner = t; break; }
            seen += counts[t];
        }
        answer[0] = owner;
        answer[1] = (int)(nth - seen);
        answer[2] = -1;
    }
    __syncthreads();
    if ((int)threadIdx.x == answer[0]) {
        int left = answer[1];
        for (int i = lo; i < hi; i++) {
            if (key_of(probs[i]) == key && --left == 0) { answer[2] = i; break; }
        }
    }
    __syncthreads();
    return answer[2];
}

__global__ void __launch_bounds__(SAMPLE_THREADS) sample_rows_kernel(
    const float* __restrict__ logits, const float* __restrict__ temperature, const int32_t* __restrict__ top_k,
    const float* __restrict__ top_p, const double* __restrict__ uniform, float* __restrict__ probs_all,
    int32_t* __restrict__ out, int vocab) {
    __shared__ float scratch[32];
    __shared__ double dscratch[32];
    __shared__ unsigned int h_cnt[256];
    __shared__ unsigned long long h_mass[256];
    __shared__ unsigned int counts[SAMPLE_THREADS];
    __shared__ Prefix result;
    __shared__ int answer[3];
    __shared__ int best_id;

    const int r = blockIdx.x, tid = threadIdx.x;
    const float* l = logits + (size_t)r * vocab;
    float* probs = probs_all + (size_t)r * vocab;
    const float temp = temperature[r];

    float mx = -INFINITY;
    for (int i = tid; i < vocab; i += blockDim.x) mx = fmaxf(mx, l[i]);
    mx = block_max(mx, scratch);

    if (!(temp > 0.0f)) {
        // greedy: the lowest id among the maxima (engine/src/sampler.c:31-38)
        if (tid == 0) best_id = vocab;
        __syncthreads();
        int mine = vocab;
        for (int i = tid; i < vocab; i += blockDim.x)
            if (l[i] == mx && i < mine) mine = i;
        if (mine < vocab) atomicMin(&best_id, mine);
        __syncthreads();
        if (tid == 0) out[r] = best_id < vocab ? best_id : 0;  // all-NaN rows fall back to id 0
        return;
    }

    double sum = 0.0;
    for (int i = tid; i < vocab; i += blockDim.x) {
        const float p = expf((l[i] - mx) / temp);
        probs[i] = p;
        sum += (double)p;
    }
    {   // block sum in double, fixed tree
        const int lane = tid & 31, warp = tid >> 5;
        for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
        if (lane == 0) dscratch[warp] = sum;
        __syncthreads();
        double s = (lane < (int)(blockDim.x >> 5)) ? dscratch[lane] : 0.0;
        for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
        sum = s;
    }
    for (int i = tid; i < vocab; i += blockDim.x) probs[i] = (float)((double)probs[i] / sum);
    __syncthreads();

    // mass of everything, exact in fixed point
    unsigned long long keep = (unsigned long long)vocab;
    const int k = top_k[r];
    const float pp = top_p[r];
    Prefix kept;
    // count-only pass when top-k cuts, else a pass to the end for the total mass
    if (k > 0 && k < vocab) keep = (unsigned long long)k;
    kept = find_prefix(probs, vocab, 0, 0ull, keep, h_cnt, h_mass, &result);
    __syncthreads();
    if (pp > 0.0f && pp < 1.0f) {
        const unsigned long long target = (unsigned long long)((double)pp * (double)kept.mass);
        kept = find_prefix(probs, vocab, 1, target, kept.count, h_cnt, h_mass, &result);
        __syncthreads();
    }
    const unsigned long long target = (unsigned long long)(uniform[r] * (double)kept.mass);
    const Prefix pick = find_prefix(probs, vocab, 2, target, kept.count, h_cnt, h_mass, &result);
    __syncthreads();
    const int id = find_nth_with_key(probs, vocab, pick.key, pick.nth, counts, answer);
    if (tid == 0) out[r] = id >= 0 ? id : 0;
}

// Greedy only: ids[r] = lowest id of the maximum of logits[r, :].  A row is shared by `parts` blocks (grid.y);
// each packs its best (value, id) into one 64-bit key whose order is "larger value first, then lower id" and
// folds it into the row's slot with atomicMax; the slot starts at zero (the host clears it on the stream) and the
// block that arrives last writes the id and leaves the slot zero for the next launch.
__device__ __forceinline__ unsigned long long argmax_key(float v, int id) {
    uint32_t b = __float_as_uint(v + 0.0f);                   // -0 becomes +0: equal values, equal keys
    b = (b & 0x80000000u) ? ~b : (b | 0x80000000u);          // order-preserving map of float32 to unsigned
    return ((unsigned long long)b << 32) | (uint32_t)(0x7fffffff - id);
}

__global__ void __launch_bounds__(256) argmax_rows_kernel(const float* __restrict__ logits, int32_t* __restrict__ out,
                                                          unsigned long long* __restrict__ slots, int* __restrict__ arrived, int vocab) {
    __shared__ unsigned long long wbest[8];
    const int r = blockIdx.x, part = blockIdx.y, parts = gridDim.y, tid = threadIdx.x;
    dependency_wait();
    const float* l = logits + (size_t)r * vocab;
    const int per = (vocab + parts - 1) / parts;
    const int lo = part * per, hi = min(vocab, lo + per);
    unsigned long long best = 0;                              // below every real key (a NaN maps above or below, never 0... ids keep it distinct)
    for (int i = lo + tid; i < hi; i += 256) {
        const unsigned long long k = argmax_key(l[i], i);
        best = k > best ? k : best;
    }
    for (int o = 16; o > 0; o >>= 1) {
        const unsigned long long other = __shfl_xor_sync(0xffffffffu, best, o);
        best = other > best ? other : best;
    }
    if ((tid & 31) == 0) wbest[tid >> 5] = best;
    __syncthreads();
    if (tid == 0) {
        for (int w = 1; w < 8; w++) best = wbest[w] > best ? wbest[w] : best;
        atomicMax(&slots[r], best);
        __threadfence();
        if (atomicAdd(&arrived[r], 1) == parts - 1) {
            __threadfence();
            const unsigned long long k = atomicExch(&slots[r], 0ull);
            out[r] = k ? (int)(0x7fffffff - (uint32_t)(k & 0xffffffffu)) : 0;
            arrived[r] = 0;
        }
    }
}

}  // namespace vk

using namespace vk;

// scratch: rows * 12 bytes (a 64-bit slot and an arrival counter per row), zero before the first launch; the kernel
// leaves it zero.
VK_API int vk_argmax_rows(const float* logits, int32_t* out, void* scratch, int rows, int vocab, cudaStream_t stream) {
    if (rows <= 0) return VK_OK;
    if (vocab <= 0 || !scratch) return VK_BAD_SHAPE;
    if ((uintptr_t)scratch % 8) return VK_BAD_ALIGNMENT;
    // enough blocks a row to use the machine: about 4096 columns each, at most 32 parts
    int parts = (vocab + 4095) / 4096;
    parts = parts < 1 ? 1 : (parts > 32 ? 32 : parts);
    unsigned long long* slots = (unsigned long long*)scratch;
    int* arrived = (int*)(slots + rows);
    return launch_dependent(argmax_rows_kernel, dim3(rows, parts), dim3(256), 0, stream, logits, out, slots, arrived, vocab);
}

// probs: scratch [rows, vocab] float32.  temperature <= 0 on a row means greedy for that row.
VK_API int vk_sample_rows(const float* logits, const float* temperature, const int32_t* top_k, const float* top_p,
                          const double* uniform, float* probs, int32_t* out, int rows, int vocab, cudaStream_t stream) {
    if (rows <= 0) return VK_OK;
    if (vocab <= 0) return VK_BAD_SHAPE;
    sample_rows_kernel<<<rows, SAMPLE_THREADS, 0, stream>>>(logits, temperature, top_k, top_p, uniform, probs, out, vocab);
    return launch_status();
}
