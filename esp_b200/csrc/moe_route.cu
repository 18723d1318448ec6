// Routing for the sparse feed-forward block: router logits, softmax, top-k and
// the shared expert's sigmoid gate in 32-bit; the permutation of (token, rank)
// pairs into expert order; and the ordered sum that brings expert outputs back
// to token order.  Nothing here returns to the host.
#include "common.cuh"

namespace {
constexpr int ROUTER_THREADS = 512;
constexpr int MAX_TOPK = 32;
constexpr int ROUTE_SMALL_MAX = 64;          // tokens of a step that the two-launch router takes (an expert's rows stay one tile)

// A lane's share of dot(hs[t], w) for TPB token rows at once: 4 consecutive
// weights at a time (8-byte loads of bfloat16, 16-byte of float), lanes
// interleaved so that the float4 reads of hs fall into distinct banks, several
// loads in flight; each weight is loaded once and used for every row.  The
// order of a lane's additions depends on the width alone.
__device__ __forceinline__ float4 load4(const bf16* w) {
    const uint2 v = *reinterpret_cast<const uint2*>(w);
    return make_float4(__uint_as_float(v.x << 16), __uint_as_float(v.x & 0xffff0000u), __uint_as_float(v.y << 16),
                       __uint_as_float(v.y & 0xffff0000u));
}
__device__ __forceinline__ float4 load4(const float* w) { return *reinterpret_cast<const float4*>(w); }

template <int TPB, typename TW>
__device__ __forceinline__ void lane_dots(const float* __restrict__ hs, int hs_stride, const TW* __restrict__ w, int width,
                                          int lane, float (&s)[TPB]) {
#pragma unroll
    for (int t = 0; t < TPB; t++) s[t] = 0.f;
    const int vec_end = (width % 4 == 0 && (reinterpret_cast<uintptr_t>(w) & 15) == 0) ? width : 0;
#pragma unroll 4
    for (int i = lane * 4; i < vec_end; i += 128) {
        const float4 f = load4(w + i);
#pragma unroll
        for (int t = 0; t < TPB; t++) {
            const float4 x = *reinterpret_cast<const float4*>(hs + t * hs_stride + i);
            s[t] = fmaf(x.x, f.x, s[t]);
            s[t] = fmaf(x.y, f.y, s[t]);
            s[t] = fmaf(x.z, f.z, s[t]);
            s[t] = fmaf(x.w, f.w, s[t]);
        }
    }
    for (int i = vec_end + lane; i < width; i += 32) {
        const float wv = to_f32(w[i]);
#pragma unroll
        for (int t = 0; t < TPB; t++) s[t] = fmaf(hs[t * hs_stride + i], wv, s[t]);
    }
}

// One block per TPB tokens.  logits[e] = sum_k h[k] * Wr[e][k]: a warp per expert,
// lanes stride over k, partial sums combined by the fixed warp butterfly.
// p = softmax(logits) over all experts; the k largest p win, ties to the lower
// id; weights are p / (sum of the chosen p) if norm_topk else p.
// gate[n] = sigmoid(h . w_gate) when w_gate is given.
template <typename TH, typename TW, int TPB>
__global__ void __launch_bounds__(ROUTER_THREADS)
router_topk_kernel(const TH* __restrict__ h, const TW* __restrict__ w_router, const TW* __restrict__ w_gate,
                   int* __restrict__ topk_ids, float* __restrict__ topk_w, float* __restrict__ gate,
                   float* __restrict__ probs_out, int n_tokens, int width, int n_experts, int top_k, int norm_topk,
                   int* __restrict__ status) {
    extern __shared__ float smem[];
    float* hs = smem;                          // [TPB][width]
    float* ps_all = smem + TPB * width;        // [TPB][n_experts]
    const int n0 = blockIdx.x * TPB, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nwarp = ROUTER_THREADS / 32;
    const int live = min(TPB, n_tokens - n0);
    for (int i = tid; i < TPB * width; i += ROUTER_THREADS) {
        const int t = i / width;
        hs[i] = t < live ? to_f32(h[(size_t)n0 * width + i]) : 0.f;
    }
    __syncthreads();
    // Each warp takes EPW experts at a time and, for every chunk of four columns, holds the TPB rows' values
    // in registers while it walks its experts: a weight is loaded once per block and a row value once
    // per EPW experts.  A lane's additions per (expert, row) run in column order.
    constexpr int EPW = 4;
    const int rows = n_experts + (w_gate ? 1 : 0);
    const bool vec = width % 4 == 0 && (reinterpret_cast<uintptr_t>(w_router) & 15) == 0 &&
                     (!w_gate || (reinterpret_cast<uintptr_t>(w_gate) & 15) == 0) && (width * sizeof(TW)) % 16 == 0;
    for (int e0 = warp * EPW; e0 < rows; e0 += nwarp * EPW) {
        float acc[EPW][TPB];
#pragma unroll
        for (int j = 0; j < EPW; j++)
#pragma unroll
            for (int t = 0; t < TPB; t++) acc[j][t] = 0.f;
        const TW* wrow[EPW];
#pragma unroll
        for (int j = 0; j < EPW; j++) {
            const int e = min(e0 + j, rows - 1);
            wrow[j] = e < n_experts ? w_router + (size_t)e * width : w_gate;
        }
        if (vec) {
#pragma unroll 2
            for (int i = lane * 4; i < width; i += 128) {
                float4 x[TPB];
#pragma unroll
                for (int t = 0; t < TPB; t++) x[t] = *reinterpret_cast<const float4*>(hs + t * width + i);
#pragma unroll
                for (int j = 0; j < EPW; j++) {
                    const float4 f = load4(wrow[j] + i);
#pragma unroll
                    for (int t = 0; t < TPB; t++) {
                        acc[j][t] = fmaf(x[t].x, f.x, acc[j][t]);
                        acc[j][t] = fmaf(x[t].y, f.y, acc[j][t]);
                        acc[j][t] = fmaf(x[t].z, f.z, acc[j][t]);
                        acc[j][t] = fmaf(x[t].w, f.w, acc[j][t]);
                    }
                }
            }
        } else {
            for (int i = lane; i < width; i += 32)
#pragma unroll
                for (int j = 0; j < EPW; j++) {
                    const float wv = to_f32(wrow[j][i]);
#pragma unroll
                    for (int t = 0; t < TPB; t++) acc[j][t] = fmaf(hs[t * width + i], wv, acc[j][t]);
                }
        }
#pragma unroll
        for (int j = 0; j < EPW; j++) {
            const int e = e0 + j;
#pragma unroll
            for (int t = 0; t < TPB; t++) {
                const float v = warp_sum(acc[j][t]);
                if (lane == 0 && t < live && e < rows) {
                    if (e < n_experts) ps_all[t * n_experts + e] = v;
                    else gate[n0 + t] = 1.0f / (1.0f + expf(-v));
                }
            }
        }
    }
    __syncthreads();
    // softmax, top-k and weights: one warp per token row, everything at warp level
    for (int t = warp; t < live; t += nwarp) {
        const int n = n0 + t;
        float* ps = ps_all + t * n_experts;
        float mx = -INFINITY;
        for (int e = lane; e < n_experts; e += 32) mx = fmaxf(mx, ps[e]);
        mx = warp_max(mx);
        float sum = 0.f;
        for (int e = lane; e < n_experts; e += 32) {
            const float p = expf(ps[e] - mx);
            ps[e] = p;
            sum += p;
        }
        sum = warp_sum(sum);
        __syncwarp();
        for (int e = lane; e < n_experts; e += 32) {
            const float p = ps[e] / sum;
            ps[e] = p;
            if (probs_out) probs_out[(size_t)n * n_experts + e] = p;
        }
        __syncwarp();
        // top-k by repeated arg-max (k and E are small); ties go to the lower id; rank r is kept by lane r
        bool bad = false;
        float mass = 0.f, my_p = 0.f;
        int my_e = 0;
        for (int r = 0; r < top_k; r++) {
            float best = -INFINITY;
            int best_e = 0x7fffffff;
            for (int e = lane; e < n_experts; e += 32) {
                const float p = ps[e];
                if (!(p == p) || isinf(p)) bad = true;
                if (p > best) { best = p; best_e = e; }   // ascending e per lane: the first maximum is the lowest id
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                const float ob = __shfl_xor_sync(0xffffffffu, best, o);
                const int oe = __shfl_xor_sync(0xffffffffu, best_e, o);
                if (ob > best || (ob == best && oe < best_e)) { best = ob; best_e = oe; }
            }
            if (best_e == 0x7fffffff) { best_e = 0; bad = true; }
            if (lane == 0) ps[best_e] = -1.0f;            // probabilities are >= 0: taken out of the running
            if (lane == r) { my_p = best; my_e = best_e; }
            mass += best;
            __syncwarp();
        }
        const float denom = norm_topk ? mass : 1.0f;
        if (__any_sync(0xffffffffu, bad) || !(denom > 0.f)) {
            if (lane == 0) atomicOr(status, ESP_STATUS_ROUTER_NONFINITE);
        }
        if (lane < top_k) {
            topk_ids[(size_t)n * top_k + lane] = my_e;
            topk_w[(size_t)n * top_k + lane] = my_p / denom;
        }
    }
}

// ---- many tokens, bfloat16 weights: the logits on the tensor cores, in 32-bit precision ----------------
// A float x is the sum of three bfloat16 numbers a + b + c exactly (8 bits of its 24-bit mantissa each), and a
// product of two bfloat16 numbers is exact in float, so  x . w = a . w + b . w + c . w  accumulated in float
// is a 32-bit dot product in another order of summation.  mma.sync m16n8k16: 16 tokens are the rows, 8
// experts a column tile.  A block takes 16 tokens; its eight (or four) warps take a share of the columns each
// and their partial sums are added in warp order.  logits[n, e] for e < E, and the shared gate's at e = E.
__device__ __forceinline__ unsigned pack2_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<unsigned*>(&v);
}
__device__ __forceinline__ void split3(float x0, float x1, unsigned& a, unsigned& b, unsigned& c) {
    const float a0 = __bfloat162float(__float2bfloat16_rn(x0)), a1 = __bfloat162float(__float2bfloat16_rn(x1));
    const float r0 = x0 - a0, r1 = x1 - a1;
    const float b0 = __bfloat162float(__float2bfloat16_rn(r0)), b1 = __bfloat162float(__float2bfloat16_rn(r1));
    a = pack2_bf16(a0, a1);
    b = pack2_bf16(b0, b1);
    c = pack2_bf16(r0 - b0, r1 - b1);
}
__device__ __forceinline__ void mma_16816(float (&d)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3, unsigned b0,
                                          unsigned b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

template <int NT, int KW>                                        // KW: warps that share the columns
__global__ void __launch_bounds__(KW * 32)
router_logits_mma_kernel(const float* __restrict__ h, const bf16* __restrict__ w_router, const bf16* __restrict__ w_gate,
                         float* __restrict__ logits, int n_tokens, int width, int n_experts) {
    __shared__ float part[KW - 1][16][NT * 8 + 1];               // the partial sums of warps 1..
    const int n0 = blockIdx.x * 16, warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, tg = lane & 3;
    const int rows = n_experts + (w_gate ? 1 : 0);
    const int row_a = min(n0 + g, n_tokens - 1), row_b = min(n0 + g + 8, n_tokens - 1);
    const float* xa = h + (size_t)row_a * width;
    const float* xb = h + (size_t)row_b * width;
    // this lane's weight row in every column tile (rows beyond the last read the last one; never stored)
    const bf16* wrow[NT];
#pragma unroll
    for (int t = 0; t < NT; t++) {
        const int e = min(t * 8 + g, rows - 1);
        wrow[t] = e < n_experts ? w_router + (size_t)e * width : w_gate;
    }
    float acc[NT][4];
#pragma unroll
    for (int t = 0; t < NT; t++)
#pragma unroll
        for (int i = 0; i < 4; i++) acc[t][i] = 0.f;
    // the MMA's k index may be any fixed rearrangement of the columns as long as both operands use it: of a run
    // of 32 columns this lane takes the 8 from tg * 8 on, four in each of two MMAs, so that its loads are 16 bytes
    const int share = width / KW;                                 // width is a multiple of KW * 32
#pragma unroll 2                                               // the loads of two steps are on their way together
    for (int k0 = warp * share; k0 < (warp + 1) * share; k0 += 32) {
#pragma unroll
        for (int s = 0; s < 2; s++) {
            const int k = k0 + tg * 8 + s * 4;
            const float4 va = *reinterpret_cast<const float4*>(xa + k), vb = *reinterpret_cast<const float4*>(xb + k);
            unsigned a[3][4];                                      // [part of the split][fragment register]
            split3(va.x, va.y, a[0][0], a[1][0], a[2][0]);
            split3(vb.x, vb.y, a[0][1], a[1][1], a[2][1]);
            split3(va.z, va.w, a[0][2], a[1][2], a[2][2]);
            split3(vb.z, vb.w, a[0][3], a[1][3], a[2][3]);
#pragma unroll
            for (int t = 0; t < NT; t++) {
                const uint2 wv = *reinterpret_cast<const uint2*>(wrow[t] + k);
#pragma unroll
                for (int part_i = 2; part_i >= 0; part_i--)        // the smallest part first
                    mma_16816(acc[t], a[part_i][0], a[part_i][1], a[part_i][2], a[part_i][3], wv.x, wv.y);
            }
        }
    }
    if (warp > 0) {
#pragma unroll
        for (int t = 0; t < NT; t++) {
            part[warp - 1][g][t * 8 + tg * 2] = acc[t][0];
            part[warp - 1][g][t * 8 + tg * 2 + 1] = acc[t][1];
            part[warp - 1][g + 8][t * 8 + tg * 2] = acc[t][2];
            part[warp - 1][g + 8][t * 8 + tg * 2 + 1] = acc[t][3];
        }
    }
    __syncthreads();
    if (warp == 0) {
#pragma unroll
        for (int t = 0; t < NT; t++)
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const int r = g + (i >> 1) * 8, e = t * 8 + tg * 2 + (i & 1);
                float v = acc[t][i];
#pragma unroll
                for (int w = 0; w < KW - 1; w++) v += part[w][r][e];   // in warp order
                if (n0 + r < n_tokens && e < rows) logits[(size_t)(n0 + r) * (n_experts + 1) + e] = v;
            }
    }
}

// softmax, top-k and weights of a token from its logits [n, E + 1]: one warp per token
__global__ void __launch_bounds__(256)
router_select_kernel(const float* __restrict__ logits, int* __restrict__ topk_ids, float* __restrict__ topk_w,
                     float* __restrict__ gate, float* __restrict__ probs_out, int n_tokens, int n_experts, int top_k,
                     int norm_topk, int has_gate, int* __restrict__ status) {
    extern __shared__ float sel_ps[];                               // [8 warps][n_experts]
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int n = blockIdx.x * 8 + warp;
    if (n >= n_tokens) return;
    float* ps = sel_ps + warp * n_experts;
    const float* lg = logits + (size_t)n * (n_experts + 1);
    float mx = -INFINITY;
    for (int e = lane; e < n_experts; e += 32) mx = fmaxf(mx, lg[e]);
    mx = warp_max(mx);
    float sum = 0.f;
    for (int e = lane; e < n_experts; e += 32) {
        const float p = expf(lg[e] - mx);
        ps[e] = p;
        sum += p;
    }
    sum = warp_sum(sum);
    __syncwarp();
    for (int e = lane; e < n_experts; e += 32) {
        const float p = ps[e] / sum;
        ps[e] = p;
        if (probs_out) probs_out[(size_t)n * n_experts + e] = p;
    }
    if (lane == 0 && has_gate) gate[n] = 1.0f / (1.0f + expf(-lg[n_experts]));
    __syncwarp();
    bool bad = false;
    float mass = 0.f, my_p = 0.f;
    int my_e = 0;
    for (int r = 0; r < top_k; r++) {
        float best = -INFINITY;
        int best_e = 0x7fffffff;
        for (int e = lane; e < n_experts; e += 32) {
            const float p = ps[e];
            if (!(p == p) || isinf(p)) bad = true;
            if (p > best) { best = p; best_e = e; }           // ascending e per lane: the first maximum is the lowest id
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oe = __shfl_xor_sync(0xffffffffu, best_e, o);
            if (ob > best || (ob == best && oe < best_e)) { best = ob; best_e = oe; }
        }
        if (best_e == 0x7fffffff) { best_e = 0; bad = true; }
        if (lane == 0) ps[best_e] = -1.0f;
        if (lane == r) { my_p = best; my_e = best_e; }
        mass += best;
        __syncwarp();
    }
    const float denom = norm_topk ? mass : 1.0f;
    if (__any_sync(0xffffffffu, bad) || !(denom > 0.f)) {
        if (lane == 0) atomicOr(status, ESP_STATUS_ROUTER_NONFINITE);
    }
    if (lane < top_k) {
        topk_ids[(size_t)n * top_k + lane] = my_e;
        topk_w[(size_t)n * top_k + lane] = my_p / denom;
    }
}

// ---- few tokens (decode): logits spread over many blocks, then one block routes and permutes --------
// logits[n, e] = dot(h[n], w_router[e]) for e < E and dot(h[n], w_gate) at e = E: one warp per (token,
// expert), eight experts per block, so that a step of a handful of tokens still fills the machine.
template <typename TH, typename TW>
__global__ void __launch_bounds__(256)
router_logits_kernel(const TH* __restrict__ h, const TW* __restrict__ w_router, const TW* __restrict__ w_gate,
                     float* __restrict__ logits, int width, int n_experts) {
    pdl_trigger();
    extern __shared__ float hs[];
    const int n = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int rows = n_experts + (w_gate ? 1 : 0);
    const int e = blockIdx.y * 8 + warp;
    const TW* wr = e < n_experts ? w_router + (size_t)e * width : w_gate;
    // the warp's weight row does not depend on the kernel before: it is asked into L2 while that one finishes
    if (e < rows)
        for (int b = lane * 128; b < width * (int)sizeof(TW); b += 32 * 128)
            asm volatile("prefetch.global.L2 [%0];\n" ::"l"(reinterpret_cast<const char*>(wr) + b));
    pdl_wait();
    for (int i = tid; i < width; i += 256) hs[i] = to_f32(h[(size_t)n * width + i]);
    __syncthreads();
    if (e >= rows) return;
    float s[1];
    lane_dots<1>(hs, width, wr, width, lane, s);
    const float v = warp_sum(s[0]);
    if (lane == 0) logits[(size_t)n * (n_experts + 1) + e] = v;
}

// One block: a warp per token turns its logits into probabilities, picks the top k (ties to the lower
// id) and the routing weights; then the whole block builds the permutation as moe_permute_kernel does.
__global__ void __launch_bounds__(256)
route_small_kernel(const float* __restrict__ logits, int* __restrict__ topk_ids, float* __restrict__ topk_w,
                   float* __restrict__ gate, float* __restrict__ probs_out, int n_tokens, int n_experts, int top_k,
                   int norm_topk, int has_gate, int* __restrict__ offsets, int* __restrict__ perm_token,
                   float* __restrict__ perm_weight, int* __restrict__ inverse, int* __restrict__ status,
                   unsigned long long* __restrict__ distinct, int* __restrict__ tile_group, int* __restrict__ tile_row0,
                   int* __restrict__ tile_count, int* __restrict__ n_tiles) {
    pdl_trigger();
    pdl_wait();
    extern __shared__ float sm_f[];
    float* ps_all = sm_f;                                      // [8 warps][n_experts]
    int* counts = reinterpret_cast<int*>(sm_f + 8 * n_experts); // [n_experts]
    int* cursor = counts + n_experts;                           // [n_experts + 1]
    int* pair_e = cursor + n_experts + 1;                       // [n_tokens * top_k]
    float* pair_w = reinterpret_cast<float*>(pair_e + n_tokens * top_k);   // [n_tokens * top_k]
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    for (int e = tid; e < n_experts; e += 256) counts[e] = 0;
    __syncthreads();
    float* ps = ps_all + warp * n_experts;
    for (int n = warp; n < n_tokens; n += 8) {
        const float* lg = logits + (size_t)n * (n_experts + 1);
        float mx = -INFINITY;
        for (int e = lane; e < n_experts; e += 32) mx = fmaxf(mx, lg[e]);
        mx = warp_max(mx);
        float sum = 0.f;
        for (int e = lane; e < n_experts; e += 32) {
            const float p = expf(lg[e] - mx);
            ps[e] = p;
            sum += p;
        }
        sum = warp_sum(sum);
        __syncwarp();
        for (int e = lane; e < n_experts; e += 32) {
            const float p = ps[e] / sum;
            ps[e] = p;
            if (probs_out) probs_out[(size_t)n * n_experts + e] = p;
        }
        if (lane == 0 && has_gate) gate[n] = 1.0f / (1.0f + expf(-lg[n_experts]));
        __syncwarp();
        bool bad = false;
        float mass = 0.f, my_p = 0.f;
        int my_e = 0;
        for (int r = 0; r < top_k; r++) {
            float best = -INFINITY;
            int best_e = 0x7fffffff;
            for (int e = lane; e < n_experts; e += 32) {
                const float p = ps[e];
                if (!(p == p) || isinf(p)) bad = true;
                if (p > best) { best = p; best_e = e; }
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                const float ob = __shfl_xor_sync(0xffffffffu, best, o);
                const int oe = __shfl_xor_sync(0xffffffffu, best_e, o);
                if (ob > best || (ob == best && oe < best_e)) { best = ob; best_e = oe; }
            }
            if (best_e == 0x7fffffff) { best_e = 0; bad = true; }
            if (lane == 0) ps[best_e] = -1.0f;
            if (lane == r) { my_p = best; my_e = best_e; }       // top_k <= 32: rank r is kept by lane r
            mass += best;
            __syncwarp();
        }
        const float denom = norm_topk ? mass : 1.0f;
        if (__any_sync(0xffffffffu, bad) || !(denom > 0.f)) {
            if (lane == 0) atomicOr(status, ESP_STATUS_ROUTER_NONFINITE);
        }
        if (lane < top_k) {
            const float w = my_p / denom;
            topk_ids[(size_t)n * top_k + lane] = my_e;
            topk_w[(size_t)n * top_k + lane] = w;
            pair_e[n * top_k + lane] = my_e;                      // kept in shared memory for the placement below
            pair_w[n * top_k + lane] = w;
            atomicAdd(&counts[my_e], 1);
        }
        __syncwarp();
    }
    __syncthreads();
    if (warp == 0) {
        // first rows of the experts' ranges: a running sum over the counts, 32 experts at a time
        int run = 0, used = 0;
        for (int e0 = 0; e0 < n_experts; e0 += 32) {
            const int e = e0 + lane;
            const int c = e < n_experts ? counts[e] : 0;
            int incl = c;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const int up = __shfl_up_sync(0xffffffffu, incl, o);
                if (lane >= o) incl += up;
            }
            if (e < n_experts) {
                cursor[e] = run + incl - c;
                offsets[e] = run + incl - c;
            }
            const unsigned with_rows = __ballot_sync(0xffffffffu, c > 0);
            // the row tiles of the grouped tensor-core products: a token names an expert once, so an expert has
            // at most as many rows as the step has tokens (at most ROUTE_SMALL_MAX) and is one tile
            if (tile_group && c > 0) {
                const int t = used + __popc(with_rows & ((1u << lane) - 1));
                tile_group[t] = e;
                tile_row0[t] = run + incl - c;
                tile_count[t] = c;
            }
            used += __popc(with_rows);
            run += __shfl_sync(0xffffffffu, incl, 31);
        }
        if (lane == 0) {
            cursor[n_experts] = run;
            offsets[n_experts] = run;
            if (n_tiles) *n_tiles = used;
            if (distinct) atomicAdd(distinct, (unsigned long long)used);     // experts that this step reads
        }
    }
    __syncthreads();
    const int n_pairs = n_tokens * top_k;
    for (int i = tid; i < n_pairs; i += 256) {
        const int e = pair_e[i];
        const int row = atomicAdd(&cursor[e], 1);
        perm_token[row] = i / top_k;
        perm_weight[row] = pair_w[i];
        inverse[i] = row;
    }
}

// The same for many pairs: every warp of the one block counts into a table of its own, so that an expert
// that takes most of the tokens is not one address that a thousand threads add to in turn; a scan over
// the warps gives every warp its first row in every expert's range, and the warp places its pairs there.
// shared memory: [32 warps][n_experts] counts, then [n_experts + 1] offsets.
__global__ void __launch_bounds__(1024)
moe_permute_wide_kernel(const int* __restrict__ topk_ids, const float* __restrict__ topk_w, int n_pairs, int n_experts,
                        int* __restrict__ offsets, int* __restrict__ perm_token, float* __restrict__ perm_weight,
                        int* __restrict__ inverse, int top_k, int* __restrict__ tile_group, int* __restrict__ tile_row0,
                        int* __restrict__ tile_count, int* __restrict__ n_tiles, int tile_rows, int max_tiles,
                        int* __restrict__ status, unsigned long long* __restrict__ distinct) {
    extern __shared__ int sm[];
    int* hist = sm;                                  // [32][n_experts]: counts, later each warp's next row
    int* offs = sm + 32 * n_experts;                 // [n_experts + 1]
    const int tid = threadIdx.x, warp = tid >> 5;
    for (int i = tid; i < 32 * n_experts; i += 1024) hist[i] = 0;
    __syncthreads();
    int* mine = hist + warp * n_experts;
    // pair i belongs to warp (i / 32) % 32 in both passes.  A thread's first PER pairs stay in registers: their loads
    // go out together (one trip to memory, not one per pair) and the second pass does not load them again.
    constexpr int PER = 8;
    int held[PER];
#pragma unroll
    for (int j = 0; j < PER; j++) {
        const int i = tid + j * 1024;
        held[j] = i < n_pairs ? topk_ids[i] : -2;
    }
#pragma unroll
    for (int j = 0; j < PER; j++) {
        if (held[j] == -2) continue;
        if (held[j] >= 0 && held[j] < n_experts) atomicAdd(&mine[held[j]], 1);
        else atomicOr(status, ESP_STATUS_BAD_INDEX);
    }
    for (int i = tid + PER * 1024; i < n_pairs; i += 1024) {
        const int e = topk_ids[i];
        if (e >= 0 && e < n_experts) atomicAdd(&mine[e], 1);
        else atomicOr(status, ESP_STATUS_BAD_INDEX);
    }
    __syncthreads();
    // thread e: the expert's total, and every warp's count turned into its share's first row within the expert
    for (int e = tid; e < n_experts; e += 1024) {
        int run = 0;
        for (int w = 0; w < 32; w++) {
            const int c = hist[w * n_experts + e];
            hist[w * n_experts + e] = run;
            run += c;
        }
        offs[e + 1] = run;                           // the total, for the scan below
    }
    __syncthreads();
    if (tid == 0) {                                  // exclusive scan in place: offs[e + 1] holds expert e's total until
        int run = 0, used = 0;                       // turn e reads it; turn e + 1 overwrites it with expert e + 1's start
        for (int e = 0; e < n_experts; e++) {
            const int c = offs[e + 1];
            offs[e] = run;
            offsets[e] = run;
            run += c;
            used += c > 0;
        }
        offs[n_experts] = run;
        offsets[n_experts] = run;
        if (distinct) atomicAdd(distinct, (unsigned long long)used);
    }
    __syncthreads();
    if (tile_group && tid == 0) {                    // row tiles of the grouped products: a tile never mixes two experts
        int t = 0;
        for (int e = 0; e < n_experts; e++) {
            const int lo = offs[e], cnt = offs[e + 1] - lo;
            for (int r = 0; r < cnt && t < max_tiles; r += tile_rows, t++) {
                tile_group[t] = e;
                tile_row0[t] = lo + r;
                tile_count[t] = min(tile_rows, cnt - r);
            }
        }
        *n_tiles = t;
    }
    float wheld[PER];
#pragma unroll
    for (int j = 0; j < PER; j++) {
        const int i = tid + j * 1024;
        wheld[j] = i < n_pairs ? topk_w[i] : 0.f;
    }
#pragma unroll
    for (int j = 0; j < PER; j++) {
        const int i = tid + j * 1024, e = held[j];
        if (e == -2) continue;
        if (e < 0 || e >= n_experts) { inverse[i] = -1; continue; }
        const int row = offs[e] + atomicAdd(&mine[e], 1);
        perm_token[row] = i / top_k;
        perm_weight[row] = wheld[j];
        inverse[i] = row;
    }
    for (int i = tid + PER * 1024; i < n_pairs; i += 1024) {
        const int e = topk_ids[i];
        if (e < 0 || e >= n_experts) { inverse[i] = -1; continue; }
        const int row = offs[e] + atomicAdd(&mine[e], 1);
        perm_token[row] = i / top_k;
        perm_weight[row] = topk_w[i];
        inverse[i] = row;
    }
}

// One block.  counts -> exclusive offsets -> placement of every (token, rank)
// pair into its expert's range.  Which row of its expert's range a pair lands
// in is left to the atomics; a row's arithmetic never depends on where it sits.
__global__ void __launch_bounds__(1024)
moe_permute_kernel(const int* __restrict__ topk_ids, const float* __restrict__ topk_w, int n_pairs, int n_experts,
                   int* __restrict__ offsets, int* __restrict__ perm_token, float* __restrict__ perm_weight,
                   int* __restrict__ inverse, int top_k, int* __restrict__ tile_group, int* __restrict__ tile_row0,
                   int* __restrict__ tile_count, int* __restrict__ n_tiles, int tile_rows, int max_tiles,
                   int* __restrict__ status, unsigned long long* __restrict__ distinct) {
    extern __shared__ int sm[];
    int* counts = sm;                      // [n_experts]
    int* cursor = sm + n_experts;          // [n_experts + 1]
    for (int e = threadIdx.x; e < n_experts; e += blockDim.x) counts[e] = 0;
    __syncthreads();
    for (int i = threadIdx.x; i < n_pairs; i += blockDim.x) {
        const int e = topk_ids[i];
        if (e >= 0 && e < n_experts) atomicAdd(&counts[e], 1);
        else atomicOr(status, ESP_STATUS_BAD_INDEX);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int run = 0, used = 0;
        for (int e = 0; e < n_experts; e++) {
            cursor[e] = run;
            offsets[e] = run;
            run += counts[e];
            used += counts[e] > 0;
        }
        cursor[n_experts] = run;
        offsets[n_experts] = run;
        if (distinct) atomicAdd(distinct, (unsigned long long)used);
        // row tiles of the grouped products: a tile never mixes two experts
        if (tile_group) {
            int t = 0;
            for (int e = 0; e < n_experts; e++)
                for (int r = 0; r < counts[e] && t < max_tiles; r += tile_rows, t++) {
                    tile_group[t] = e;
                    tile_row0[t] = offsets[e] + r;
                    tile_count[t] = min(tile_rows, counts[e] - r);
                }
            *n_tiles = t;
        }
    }
    __syncthreads();
    for (int i = threadIdx.x; i < n_pairs; i += blockDim.x) {
        const int e = topk_ids[i];
        if (e < 0 || e >= n_experts) { inverse[i] = -1; continue; }
        const int row = atomicAdd(&cursor[e], 1);
        perm_token[row] = i / top_k;
        perm_weight[row] = topk_w[i];
        inverse[i] = row;
    }
}

// y[t, :] = sum over the token's chosen experts, in ascending expert id, of
// expert_out[inverse[t, r], :] (already scaled by the routing weight), then
// + gate[t] * shared[t, :].
__global__ void moe_combine_kernel(const float* __restrict__ expert_out, const int* __restrict__ topk_ids,
                                   const int* __restrict__ inverse, const float* __restrict__ gate,
                                   const float* __restrict__ shared, float* __restrict__ y, int width, int top_k) {
    pdl_trigger();
    pdl_wait();
    __shared__ int order[MAX_TOPK];
    const int t = blockIdx.x;
    if (threadIdx.x == 0) {
        int ids[MAX_TOPK];
        for (int r = 0; r < top_k; r++) { ids[r] = topk_ids[(size_t)t * top_k + r]; order[r] = r; }
        for (int a = 1; a < top_k; a++) {          // insertion sort of ranks by expert id
            const int oa = order[a], ia = ids[oa];
            int b = a - 1;
            while (b >= 0 && ids[order[b]] > ia) { order[b + 1] = order[b]; b--; }
            order[b + 1] = oa;
        }
        for (int r = 0; r < top_k; r++) order[r] = inverse[(size_t)t * top_k + order[r]];
    }
    __syncthreads();
    const float g = gate ? gate[t] : 0.f;
    if ((width & 3) == 0) {
        // four columns per thread; each column still adds its terms in the same order
        for (int i = threadIdx.x * 4; i < width; i += blockDim.x * 4) {
            float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
            for (int r = 0; r < top_k; r++) {
                const int row = order[r];
                if (row >= 0) {
                    const float4 v = *reinterpret_cast<const float4*>(expert_out + (size_t)row * width + i);
                    acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
                }
            }
            if (shared) {
                const float4 v = *reinterpret_cast<const float4*>(shared + (size_t)t * width + i);
                acc.x += g * v.x; acc.y += g * v.y; acc.z += g * v.z; acc.w += g * v.w;
            }
            *reinterpret_cast<float4*>(y + (size_t)t * width + i) = acc;
        }
        return;
    }
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        float acc = 0.f;
        for (int r = 0; r < top_k; r++) {
            const int row = order[r];
            if (row >= 0) acc += expert_out[(size_t)row * width + i];
        }
        if (shared) acc += g * shared[(size_t)t * width + i];
        y[(size_t)t * width + i] = acc;
    }
}
// The combine above fused with what follows it in a pre-norm block: the residual add and the next RMSNorm.
//   y = (sum of the row's expert outputs in ascending expert id) + gate * shared      (as moe_combine_kernel)
//   v = x[s] + y;  if (write_x) x[s] = v;  h[r] = v * rsqrt(mean(v^2) + eps) * gamma  (as add_rmsnorm)
// with s = rows ? rows[r] : r.  Same operations in the same order as the two separate kernels, so the
// results are the same bits.  Width a multiple of 4, at most 16384.
template <typename TH>
__global__ void __launch_bounds__(1024)
moe_combine_add_rmsnorm_kernel(const float* __restrict__ expert_out, const int* __restrict__ topk_ids,
                               const int* __restrict__ inverse, const float* __restrict__ gate,
                               const float* __restrict__ shared, float* __restrict__ x, const float* __restrict__ gamma,
                               const int* __restrict__ rows, TH* __restrict__ h, float* __restrict__ h32, int width,
                               int top_k, float eps, int write_x, int early) {
    pdl_trigger();
    // The kernel before this one in the stream made the experts' rows or the shared expert's row.  It lets this one
    // be set up only behind its own wait (the grouped product gives its signal when its weights are in), and by then
    // the kernels before it have ended: the routing, the gate and the residual row are complete and are read before
    // the wait, while that kernel finishes.  ``early`` 0 (every grouped product a dependent launch): everything waits.
    if (!early) pdl_wait();
    __shared__ int order[MAX_TOPK];
    __shared__ float scratch[33];
    const int r = blockIdx.x;
    const size_t t = rows ? (size_t)rows[r] : (size_t)r;
    if (threadIdx.x == 0) {
        int ids[MAX_TOPK];
        for (int j = 0; j < top_k; j++) { ids[j] = topk_ids[t * top_k + j]; order[j] = j; }
        for (int a = 1; a < top_k; a++) {
            const int oa = order[a], ia = ids[oa];
            int b = a - 1;
            while (b >= 0 && ids[order[b]] > ia) { order[b + 1] = order[b]; b--; }
            order[b + 1] = oa;
        }
        for (int j = 0; j < top_k; j++) order[j] = inverse[t * top_k + order[j]];
    }
    const float g = gate ? gate[t] : 0.f;
    const int pieces = width / 4;
    float4 v[4];
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const int q = threadIdx.x + i * blockDim.x;
        if (q < pieces) v[i] = reinterpret_cast<float4*>(x + t * width)[q];
    }
    __syncthreads();
    pdl_wait();
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const int q = threadIdx.x + i * blockDim.x;
        if (q < pieces) {
            float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
            for (int j = 0; j < top_k; j++) {
                const int row = order[j];
                if (row >= 0) {
                    const float4 e = reinterpret_cast<const float4*>(expert_out + (size_t)row * width)[q];
                    acc.x += e.x; acc.y += e.y; acc.z += e.z; acc.w += e.w;
                }
            }
            if (shared) {
                const float4 e = reinterpret_cast<const float4*>(shared + t * width)[q];
                acc.x += g * e.x; acc.y += g * e.y; acc.z += g * e.z; acc.w += g * e.w;
            }
            float4 xv = v[i];
            xv.x += acc.x; xv.y += acc.y; xv.z += acc.z; xv.w += acc.w;
            if (write_x) reinterpret_cast<float4*>(x + t * width)[q] = xv;
            v[i] = xv;
            ss = fmaf(xv.x, xv.x, ss);
            ss = fmaf(xv.y, xv.y, ss);
            ss = fmaf(xv.z, xv.z, ss);
            ss = fmaf(xv.w, xv.w, ss);
        }
    }
    const float total = block_sum(ss, scratch);
    const float inv = 1.0f / sqrtf(total / (float)width + eps);
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const int q = threadIdx.x + i * blockDim.x;
        if (q < pieces) {
            const float4 gm = reinterpret_cast<const float4*>(gamma)[q];
            const float o0 = v[i].x * inv * gm.x, o1 = v[i].y * inv * gm.y, o2 = v[i].z * inv * gm.z, o3 = v[i].w * inv * gm.w;
            TH* hr = h + (size_t)r * width + 4 * q;
            Vec4<TH>::store(hr, o0, o1, o2, o3);
            if (h32) reinterpret_cast<float4*>(h32 + (size_t)r * width)[q] = make_float4(o0, o1, o2, o3);
        }
    }
}
}  // namespace

// ``logits`` (may be null): scratch [n_tokens, n_experts + 1] float.  With it, 32-bit activations, bfloat16
// weights, many tokens and a width that is a multiple of 128, the logits are made on the tensor cores.
ESP_API int esp_router_topk(const void* h, int h_is_bf16, const void* w_router, const void* w_gate, int w_is_bf16,
                            int* topk_ids, float* topk_w, float* gate, float* probs_out, float* logits, int n_tokens,
                            int width, int n_experts, int top_k, int norm_topk, int* status, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (top_k > MAX_TOPK || top_k <= 0 || top_k > n_experts) return (int)cudaErrorInvalidValue;
    const int rows = n_experts + (w_gate ? 1 : 0);
    if (logits && !h_is_bf16 && w_is_bf16 && n_tokens >= 64 && width % 128 == 0 && rows <= 72 &&
        (size_t)8 * n_experts * sizeof(float) <= 48 * 1024 && (reinterpret_cast<uintptr_t>(h) & 15) == 0 &&
        (reinterpret_cast<uintptr_t>(w_router) & 7) == 0 && (!w_gate || (reinterpret_cast<uintptr_t>(w_gate) & 7) == 0)) {
        const int blocks = (n_tokens + 15) / 16;
#define ESP_ROUTER_MMA(NT, KW)                                                                                         \
    router_logits_mma_kernel<NT, KW><<<blocks, KW * 32, 0, stream>>>((const float*)h, (const bf16*)w_router,            \
                                                                      (const bf16*)w_gate, logits, n_tokens, width, n_experts)
        if (width % 256 == 0) {
            if (rows <= 64) ESP_ROUTER_MMA(8, 8);
            else ESP_ROUTER_MMA(9, 8);
        } else {
            if (rows <= 64) ESP_ROUTER_MMA(8, 4);
            else ESP_ROUTER_MMA(9, 4);
        }
#undef ESP_ROUTER_MMA
        router_select_kernel<<<(n_tokens + 7) / 8, 256, (size_t)8 * n_experts * sizeof(float), stream>>>(
            logits, topk_ids, topk_w, gate, probs_out, n_tokens, n_experts, top_k, norm_topk, w_gate ? 1 : 0, status);
        return esp_launch_status();
    }
    // many tokens: four or eight per block, so that the router's weights are fetched that much less often
    int tpb = n_tokens > 256 ? 8 : n_tokens > 32 ? 4 : 1;
    if ((size_t)tpb * (width + n_experts) * sizeof(float) > 200 * 1024) tpb = 1;
    const size_t smem = (size_t)tpb * (width + n_experts) * sizeof(float);
    if (smem > 200 * 1024) return (int)cudaErrorInvalidValue;
    const int blocks = (n_tokens + tpb - 1) / tpb;
#define ESP_ROUTER(TH, TW, TPB)                                                                                       \
    do {                                                                                                              \
        if (smem > 48 * 1024)                                                                                         \
            cudaFuncSetAttribute(router_topk_kernel<TH, TW, TPB>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
        router_topk_kernel<TH, TW, TPB><<<blocks, ROUTER_THREADS, smem, stream>>>(                                     \
            (const TH*)h, (const TW*)w_router, (const TW*)w_gate, topk_ids, topk_w, gate, probs_out, n_tokens, width, \
            n_experts, top_k, norm_topk, status);                                                                     \
    } while (0)
#define ESP_ROUTER_T(TH, TW)                                                                                          \
    do {                                                                                                              \
        if (tpb == 8) ESP_ROUTER(TH, TW, 8);                                                                          \
        else if (tpb == 4) ESP_ROUTER(TH, TW, 4);                                                                     \
        else ESP_ROUTER(TH, TW, 1);                                                                                   \
    } while (0)
    if (h_is_bf16 && w_is_bf16) ESP_ROUTER_T(bf16, bf16);
    else if (h_is_bf16) ESP_ROUTER_T(bf16, float);
    else if (w_is_bf16) ESP_ROUTER_T(float, bf16);
    else ESP_ROUTER_T(float, float);
#undef ESP_ROUTER_T
#undef ESP_ROUTER
    return esp_launch_status();
}

// Router and permutation for a step of few tokens (at most ROUTE_SMALL_MAX) in two launches.  ``logits`` is scratch
// [n_tokens, n_experts + 1] float.  tile_group / tile_row0 / tile_count / n_tiles (may be null): the list of row
// tiles for the grouped tensor-core products, as esp_moe_permute makes it (here: one tile per expert with rows).
ESP_API int esp_route_small(const void* h, int h_is_bf16, const void* w_router, const void* w_gate, int w_is_bf16,
                            float* logits, int* topk_ids, float* topk_w, float* gate, float* probs_out, int n_tokens,
                            int width, int n_experts, int top_k, int norm_topk, int* offsets, int* perm_token,
                            float* perm_weight, int* inverse, int* status, unsigned long long* distinct, int* tile_group,
                            int* tile_row0, int* tile_count, int* n_tiles, int max_tiles, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (top_k > MAX_TOPK || top_k <= 0 || top_k > n_experts || n_tokens > ROUTE_SMALL_MAX) return (int)cudaErrorInvalidValue;
    // the tile list (all four or none): one tile per expert with rows
    if (tile_group && (!tile_row0 || !tile_count || !n_tiles || max_tiles < (n_experts < n_tokens * top_k ? n_experts : n_tokens * top_k)))
        return (int)cudaErrorInvalidValue;
    const size_t smem_a = (size_t)width * sizeof(float);
    const size_t smem_b = (size_t)(8 * n_experts) * sizeof(float) + (size_t)(2 * n_experts + 1) * sizeof(int) +
                          (size_t)n_tokens * top_k * (sizeof(int) + sizeof(float));
    if (smem_a > 48 * 1024 || smem_b > 48 * 1024) return (int)cudaErrorInvalidValue;
    const dim3 grid(n_tokens, (n_experts + 1 + 7) / 8);
#define ESP_LOGITS(TH, TW)                                                                                        \
    esp_launch_pdl(ESP_PDL_SMALL, router_logits_kernel<TH, TW>, dim3(grid), dim3(256), smem_a, stream, (const TH*)h, (const TW*)w_router, (const TW*)w_gate, \
                                                                logits, width, n_experts)
    if (h_is_bf16 && w_is_bf16) ESP_LOGITS(bf16, bf16);
    else if (h_is_bf16) ESP_LOGITS(bf16, float);
    else if (w_is_bf16) ESP_LOGITS(float, bf16);
    else ESP_LOGITS(float, float);
#undef ESP_LOGITS
    esp_launch_pdl(ESP_PDL_SMALL, route_small_kernel, dim3(1), dim3(256), smem_b, stream, logits, topk_ids, topk_w, gate, probs_out, n_tokens, n_experts, top_k,
                                                   norm_topk, w_gate ? 1 : 0, offsets, perm_token, perm_weight, inverse,
                                                   status, distinct, tile_group, tile_row0, tile_count, n_tiles);
    return esp_launch_status();
}

// ``distinct`` (may be null): a 64-bit counter to which the number of experts with at least one row is added.
// tile_group / tile_row0 / tile_count / n_tiles (may be null): the list of row tiles of at most
// ``tile_rows`` rows each (group, first row, rows), at most ``max_tiles`` of them (pass at least
// ceil(pairs / tile_rows) + n_experts).
ESP_API int esp_moe_permute(const int* topk_ids, const float* topk_w, int n_tokens, int top_k, int n_experts,
                            int* offsets, int* perm_token, float* perm_weight, int* inverse, int* tile_group,
                            int* tile_row0, int* tile_count, int* n_tiles, int tile_rows, int max_tiles, int* status,
                            unsigned long long* distinct, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    const size_t smem = (size_t)(2 * n_experts + 1) * sizeof(int);
    if (smem > 48 * 1024) return (int)cudaErrorInvalidValue;
    const size_t smem_wide = (size_t)(33 * n_experts + 1) * sizeof(int);
    if (n_tokens * top_k >= 2048 && smem_wide <= 48 * 1024) {
        moe_permute_wide_kernel<<<1, 1024, smem_wide, stream>>>(topk_ids, topk_w, n_tokens * top_k, n_experts, offsets,
                                                                perm_token, perm_weight, inverse, top_k, tile_group, tile_row0,
                                                                tile_count, n_tiles, tile_rows, max_tiles, status, distinct);
        return esp_launch_status();
    }
    moe_permute_kernel<<<1, 1024, smem, stream>>>(topk_ids, topk_w, n_tokens * top_k, n_experts, offsets, perm_token,
                                                  perm_weight, inverse, top_k, tile_group, tile_row0, tile_count, n_tiles,
                                                  tile_rows, max_tiles, status, distinct);
    return esp_launch_status();
}

ESP_API int esp_moe_combine(const float* expert_out, const int* topk_ids, const int* inverse, const float* gate,
                            const float* shared, float* y, int n_tokens, int width, int top_k, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (top_k > MAX_TOPK) return (int)cudaErrorInvalidValue;
    esp_launch_pdl(ESP_PDL_SMALL, moe_combine_kernel, dim3(n_tokens), dim3(256), 0, stream, expert_out, topk_ids, inverse, gate, shared, y, width, top_k);
    return esp_launch_status();
}

ESP_API int esp_moe_combine_add_rmsnorm(const float* expert_out, const int* topk_ids, const int* inverse, const float* gate,
                                        const float* shared, float* x, const float* gamma, const int* rows, void* h,
                                        int h_is_bf16, float* h32, int n_rows, int width, int top_k, float eps, int write_x,
                                        cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    if (top_k > MAX_TOPK || width % 4 != 0 || width > 16384) return (int)cudaErrorInvalidValue;
    int threads = ((width / 4 + 3) / 4 + 31) / 32 * 32;
    // one piece per thread while a block can hold them: a row's sum then has the same order whatever else is in the
    // step (the 32-bit path relies on it).  Many rows rounded to bfloat16: four pieces per thread, smaller blocks,
    // more rows in flight per SM.
    if (width / 4 <= 1024 && !(h_is_bf16 && n_rows >= 256)) threads = (width / 4 + 31) / 32 * 32;
    const int early = esp_pdl_enabled(ESP_PDL_GROUPED) ? 0 : 1;
    if (h_is_bf16)
        esp_launch_pdl(ESP_PDL_SMALL, moe_combine_add_rmsnorm_kernel<bf16>, dim3(n_rows), dim3(threads), 0, stream, expert_out, topk_ids, inverse, gate, shared, x, gamma,
                                                                            rows, (bf16*)h, h32, width, top_k, eps, write_x, early);
    else
        esp_launch_pdl(ESP_PDL_SMALL, moe_combine_add_rmsnorm_kernel<float>, dim3(n_rows), dim3(threads), 0, stream, expert_out, topk_ids, inverse, gate, shared, x,
                                                                             gamma, rows, (float*)h, h32, width, top_k, eps,
                                                                             write_x, early);
    return esp_launch_status();
}
