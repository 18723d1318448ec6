// Choosing the next token of each row of a logits matrix on the device.
//
// temperature == 0: the arg-max, lower id on ties.
// temperature  > 0: weights w_i = exp((l_i - max) / T) in 32-bit; the ids are
// ranked by descending weight, ties by ascending id; an optional nucleus cut
// keeps the shortest prefix of that ranking whose mass reaches top_p * total;
// one uniform draw u in [0, 1) from the row's splitmix64 stream picks the first
// id whose cumulative mass reaches u * (kept mass).  Exactly one draw per token.
//
// The ranking is never materialised: the crossing point is found by a radix
// selection over the 64-bit key (~bits(w) << 32 | id), eight passes of eight
// bits, each pass summing the mass of every bucket.  Masses are summed as
// 40-bit fixed point integers, so the sums are exact and do not depend on the
// order in which threads add them.
#include "common.cuh"

namespace {
constexpr int PICK_THREADS = 1024;
constexpr float FIXED_ONE = 1099511627776.0f;   // 2^40

__device__ __forceinline__ unsigned long long splitmix_next(unsigned long long* state) {
    *state += 0x9E3779B97F4A7C15ull;
    unsigned long long z = *state;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}

struct SelectResult {
    int id;
    unsigned long long mass_inclusive;
};

// All threads of the block call this together.  Finds the first id, in ranking
// order, whose cumulative mass is >= threshold (the last ranked id with any
// mass if the threshold is never reached).
__device__ SelectResult select_crossing(const float* __restrict__ row, int vocab, float mx, float inv_t,
                                        unsigned long long threshold, unsigned long long* hist, int* bucket_count,
                                        unsigned long long* shared_out) {
    unsigned long long prefix = 0, mask = 0, before = 0;
    for (int byte = 7; byte >= 0; byte--) {
        const int shift = 8 * byte;
        for (int b = threadIdx.x; b < 256; b += blockDim.x) { hist[b] = 0; bucket_count[b] = 0; }
        __syncthreads();
        for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
            const float w = expf((row[i] - mx) * inv_t);
            const unsigned long long key = ((unsigned long long)(~__float_as_uint(w)) << 32) | (unsigned)i;
            if ((key & mask) == prefix) {
                const int b = (int)((key >> shift) & 255ull);
                atomicAdd(&hist[b], (unsigned long long)__float2ull_rd(w * FIXED_ONE));
                atomicAdd(&bucket_count[b], 1);
            }
        }
        __syncthreads();
        if (threadIdx.x == 0) {
            int pick = -1, last = -1;
            unsigned long long run = before, before_last = before;
            for (int b = 0; b < 256; b++) {
                if (bucket_count[b] == 0) continue;
                last = b;
                before_last = run;
                if (hist[b] > 0 && run + hist[b] >= threshold) { pick = b; break; }
                run += hist[b];
            }
            if (pick < 0) { pick = last < 0 ? 0 : last; run = before_last; }
            shared_out[0] = (unsigned long long)pick;
            shared_out[1] = run;
        }
        __syncthreads();
        prefix |= shared_out[0] << shift;
        mask |= 255ull << shift;
        before = shared_out[1];
        __syncthreads();
    }
    SelectResult r;
    r.id = (int)(prefix & 0xffffffffull);
    if (r.id < 0 || r.id >= vocab) r.id = vocab - 1;
    const float w = expf((row[r.id] - mx) * inv_t);
    r.mass_inclusive = before + (unsigned long long)__float2ull_rd(w * FIXED_ONE);
    return r;
}

__global__ void __launch_bounds__(PICK_THREADS)
pick_tokens_kernel(const float* __restrict__ logits, int vocab, const float* __restrict__ temperature,
                   const float* __restrict__ top_p, unsigned long long* __restrict__ rng_state,
                   const int* __restrict__ row_slot, int* __restrict__ tokens) {
    pdl_trigger();
    pdl_wait();
    __shared__ float best_v[PICK_THREADS / 32];
    __shared__ int best_i[PICK_THREADS / 32];
    __shared__ unsigned long long hist[256];
    __shared__ int bucket_count[256];
    __shared__ unsigned long long shared_out[2];
    const int r = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const float* row = logits + (size_t)r * vocab;
    const float temp = temperature ? temperature[r] : 0.f;

    // arg-max with the lower id on ties (also gives the maximum for the weights)
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    for (int i = tid; i < vocab; i += PICK_THREADS) {
        const float v = row[i];
        if (v > bv) { bv = v; bi = i; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
    }
    if (lane == 0) { best_v[warp] = bv; best_i[warp] = bi; }
    __syncthreads();
    if (warp == 0) {
        bv = lane < PICK_THREADS / 32 ? best_v[lane] : -INFINITY;
        bi = lane < PICK_THREADS / 32 ? best_i[lane] : 0x7fffffff;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
        }
        if (lane == 0) { best_v[0] = bv; best_i[0] = bi == 0x7fffffff ? 0 : bi; }
    }
    __syncthreads();
    const float mx = best_v[0];
    if (!(temp > 0.f)) {
        if (tid == 0) tokens[r] = best_i[0];
        return;
    }
    const float inv_t = 1.0f / temp;
    // total mass (exact fixed-point sum)
    unsigned long long local = 0;
    for (int i = tid; i < vocab; i += PICK_THREADS) local += __float2ull_rd(expf((row[i] - mx) * inv_t) * FIXED_ONE);
    if (tid == 0) shared_out[0] = 0;
    __syncthreads();
    atomicAdd(&shared_out[0], local);
    __syncthreads();
    unsigned long long kept = shared_out[0];
    __syncthreads();
    const float tp = top_p ? top_p[r] : -1.f;
    if (tp >= 0.f) {
        const float c = fminf(fmaxf(tp, 0.f), 1.f);
        const unsigned long long target = (unsigned long long)((double)kept * (double)c);
        kept = select_crossing(row, vocab, mx, inv_t, target, hist, bucket_count, shared_out).mass_inclusive;
    }
    // one draw per token; the uniform is rounded to 32-bit before it is scaled
    if (tid == 0) {
        unsigned long long st = rng_state[row_slot[r]];
        const unsigned long long z = splitmix_next(&st);
        rng_state[row_slot[r]] = st;
        const float u = (float)((double)(z >> 11) * (1.0 / 9007199254740992.0));
        shared_out[0] = (unsigned long long)((double)u * (double)kept);
    }
    __syncthreads();
    unsigned long long threshold = shared_out[0];
    __syncthreads();
    if (threshold > kept) threshold = kept;
    const SelectResult pick = select_crossing(row, vocab, mx, inv_t, threshold, hist, bucket_count, shared_out);
    if (tid == 0) tokens[r] = pick.id;
}
}  // namespace

ESP_API int esp_pick_tokens(const float* logits, int n_rows, int vocab, const float* temperature, const float* top_p,
                            unsigned long long* rng_state, const int* row_slot, int* tokens, cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    esp_launch_pdl(ESP_PDL_SMALL, pick_tokens_kernel, dim3(n_rows), dim3(PICK_THREADS), 0, stream, logits, vocab, temperature, top_p, rng_state, row_slot, tokens);
    return esp_launch_status();
}
