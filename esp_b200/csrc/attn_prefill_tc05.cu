// Prefill attention on the 5th-generation tensor cores: causal, optionally
// windowed, grouped query heads, sequences of unequal length packed back to
// back, keys and values read from the paged bfloat16 cache.
//
// An item is 128 consecutive new tokens of one sequence and one query head; a
// block works through a run of items, and for each walks the keys the item may
// see in blocks of 128 (two pages of 64):
//
//   S  = Q K^T       tcgen05.mma, M = 128 queries, N = 128 keys, K = head size; float accumulator in TMEM
//   P  = exp2(S * log2(e) / sqrt(hd) - m)   in 32-bit, by the threads that own the row (TMEM lane = row);
//        rounded to bfloat16 and written back over S in tensor memory (two keys to a 32-bit column), where
//        the next product reads it as its A operand: P never passes through shared memory
//   PV = P V         tcgen05.mma, N = head size, K = 128 keys, a fresh accumulator per block of keys
//   O  = O * exp2(m_old - m_new) + PV        in registers of the row's thread; O / l at the end
//
// Warp 0 loads (TMA: queries once, then keys and values page by page into three-stage rings of their own:
// a key stage is free as soon as S is done, before its block's PV; a load takes longer to land than a
// block of keys takes to work through, so two blocks have to be in flight), warp 1 issues the MMAs, the other
// warps are the row threads, two to a row (four can be chosen; each takes a share of the keys of a
// block and of the head's columns: with one warp per scheduler the chain multiply, exp2, add, round would
// run at its latency).  S and PV have two TMEM buffers each (4 x 128 = all 512 columns), so S of the
// next block runs while the row threads work on this one, and the row threads wait for a PV only when they
// add it to O, a block later.  Every wait is bounded.
//
// Head sizes 64 and 128.  The page size is 64.  Rows of the tile beyond the sequence's new tokens are
// computed and not stored; keys beyond a row's position are masked before the maximum is taken.
#include "tc05.cuh"

namespace {
using namespace tc05;
constexpr int BM = 128, BN = 128, PAGE = 64;   // warps: 0 loads, 1 MMA, then 4 * ROWT warps of row threads
constexpr int ATOM_BYTES = 128 * 128;           // 128 rows of 128 bytes: one 64-wide slice of a 128-row operand
constexpr int STAGES = 3;                       // blocks of keys (and of values) in shared memory

struct AttnParams {
    bf16* out;
    const int* tile_seq;
    const int* tile_first;
    const int* seq_start;
    const int* seq_past;
    const int* block_table;
    int table_stride, n_pages, nh, nkv, window, kv_rows, n_tiles, smem_bytes;
    int* status;
};

// instruction descriptor: bfloat16 x bfloat16 -> float, M = 128, N = n, A K-major, B K-major or MN-major
__device__ __forceinline__ unsigned idesc_attn(int n, bool b_mn_major) {
    return (1u << 4) | (1u << 7) | (1u << 10) | (b_mn_major ? (1u << 16) : 0u) | ((unsigned)(n >> 3) << 17) |
           ((unsigned)(128 >> 4) << 24);
}
// descriptor of an MN-major operand: rows are 16 consecutive k (keys), 128 bytes of n (head columns) each;
// the next 64 columns lie ``lbo`` bytes further, the next 8 keys 1024 bytes further
__device__ __forceinline__ unsigned long long smem_desc_mn(const void* p, unsigned lbo) {
    unsigned long long d = 0;
    d |= (unsigned long long)((smem_u32(p) & 0x3FFFFu) >> 4);
    d |= (unsigned long long)((lbo >> 4) & 0x3FFFu) << 16;
    d |= (unsigned long long)(1024 >> 4) << 32;
    d |= (unsigned long long)1 << 46;
    d |= (unsigned long long)2 << 61;
    return d;
}

// 2^x by the special function unit (ex2.approx: relative error about 2^-22; -inf gives 0)
__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
    return y;
}
// the ``count`` threads that meet at named barrier ``id`` learn whether all of them are well
__device__ __forceinline__ bool pair_agree(bool ok, int id, int count) {
    unsigned all;
    asm volatile(
        "{\n.reg .pred p, q;\n"
        "setp.ne.u32 p, %1, 0;\n"
        "bar.red.and.pred q, %2, %3, p;\n"
        "selp.u32 %0, 1, 0, q;\n}\n"
        : "=r"(all) : "r"(ok ? 1u : 0u), "r"(id), "r"(count) : "memory");
    return all != 0;
}
__device__ __forceinline__ void named_sync(int id, int count) {
    asm volatile("bar.sync %0, %1;\n" ::"r"(id), "r"(count) : "memory");
}

// the tile of 128 query rows and the head that a block works on
struct Item {
    int seq, h, kvh, row0, rows, pos0, pos_last, blk_lo, nb;
};
__device__ __forceinline__ Item load_item(const AttnParams& p, int item) {
    Item it;
    const int tile = item / p.nh;
    it.h = item - tile * p.nh;
    it.kvh = it.h / (p.nh / p.nkv);
    it.seq = p.tile_seq[tile];
    const int first = p.tile_first[tile];
    it.row0 = p.seq_start[it.seq] + first;                               // the tile's first row among the packed tokens
    it.rows = min(BM, p.seq_start[it.seq + 1] - p.seq_start[it.seq] - first);
    it.pos0 = p.seq_past[it.seq] + first;
    it.pos_last = it.pos0 + it.rows - 1;
    const int key_lo = p.window > 0 ? max(0, it.pos0 - p.window + 1) : 0;
    it.blk_lo = key_lo / BN;
    it.nb = it.pos_last / BN - it.blk_lo + 1;
    return it;
}

// Persistent: the (tile, head) items are listed with the most keys first; block b takes the items
// b, 2G-1-b, 2G+b, 4G-1-b, ... (G blocks), so that a long item is followed by a short one.  Every role
// derives the same run of items, and the counters of key blocks (g) and items (n_items_done) that choose
// the stage, the TMEM buffer and the phase of each mbarrier run on from one item to the next.
// ROWT: threads that share a query row (2 or 4): each takes 128 / ROWT keys of a block and HD / ROWT columns of O.
template <int HD, int ROWT>
__global__ void __launch_bounds__(64 + ROWT * 128, 1)
attn_prefill_tc05_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                         const __grid_constant__ CUtensorMap map_v, AttnParams p) {
    constexpr int HALVES = HD / 64;                       // 64-column slices of a head
    constexpr int Q_BYTES = HALVES * ATOM_BYTES, KV_BYTES = HALVES * ATOM_BYTES;
    const int n_items = p.n_tiles * p.nh, G = gridDim.x;
    auto item_of = [&](int round) { return round * G + ((round & 1) ? G - 1 - (int)blockIdx.x : (int)blockIdx.x); };

    extern __shared__ __align__(1024) unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    unsigned char* q_s = smem;
    unsigned char* k_s = q_s + Q_BYTES;                   // [STAGES]
    unsigned char* v_s = k_s + STAGES * KV_BYTES;         // [STAGES]
    unsigned long long* bars = reinterpret_cast<unsigned long long*>(v_s + STAGES * KV_BYTES);
    constexpr int N_BARS = 7 + 4 * STAGES;
    unsigned long long* q_full = bars;                    // [1]
    unsigned long long* q_empty = bars + 1;               // [1]
    unsigned long long* p_ready = bars + 2;               // [1]
    unsigned long long* s_full = bars + 3;                // [2]
    unsigned long long* pv_full = bars + 5;               // [2]
    unsigned long long* k_full = bars + 7;                // [STAGES]
    unsigned long long* k_empty = k_full + STAGES;        // [STAGES]
    unsigned long long* v_full = k_empty + STAGES;        // [STAGES]
    unsigned long long* v_empty = v_full + STAGES;        // [STAGES]
    unsigned* tmem_slot = reinterpret_cast<unsigned*>(bars + N_BARS);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    static_assert(N_BARS * 8 + 8 <= 256, "the barriers and the two words after them take 256 bytes");
    float* xchg = reinterpret_cast<float*>(bars) + 64;    // [ROWT][128]: the row threads' maxima of a block, their sums at the end
    // where shared memory is too short for the slack that rounding up to 1024 bytes needs, its start has to
    // be aligned already; the block refuses to run otherwise
    if (smem + Q_BYTES + 2 * STAGES * KV_BYTES + 256 + ROWT * 128 * 4 > smem_raw + p.smem_bytes) {
        if (threadIdx.x == 0) atomicOr(p.status, ESP_STATUS_SMEM_LAYOUT);
        return;
    }

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        for (int i = 0; i < N_BARS; i++) mbar_init(&bars[i], i == 2 ? 4 * ROWT : 1);   // p_ready: one arrival per warp of row threads
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_u32(tmem_slot)), "r"(512));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::);
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const unsigned tmem_base = *tmem_slot;
    const unsigned tm_s = tmem_base, tm_pv = tmem_base + 256;          // S buffers at columns 0 and 128, PV at 256 and 384

    if (warp == 0) {
        // ---- loads: lanes 0..HALVES-1 the queries; then per block of keys, lane = (page of the block, slice)
        bool ok = true;
        const int pg_in_blk = lane / HALVES, half = lane % HALVES;      // lanes 0..2*HALVES-1 issue boxes
        int g = 0, issued_q = 0, issued_k = 0, issued_v = 0;
        for (int round = 0; ok; round++) {
            const int item = item_of(round);
            if (item >= n_items) break;
            const Item t = load_item(p, item);
            if (lane == 0) {                                             // the last item's S products have read its queries
                ok = !*abort_flag && mbar_wait(q_empty, (round & 1) ^ 1);
                if (ok) mbar_expect_tx(q_full, Q_BYTES);
            }
            ok = __shfl_sync(0xffffffffu, ok, 0);
            if (!ok) break;
            if (lane < HALVES) tma_load_2d(q_s + lane * ATOM_BYTES, &map_q, t.h * HD + lane * 64, t.row0, q_full);
            issued_q = round + 1;
            for (int j = 0; j < t.nb && ok; j++, g++) {
                const int s = g % STAGES, ph = (g / STAGES) & 1;
                // the page of this lane's box; a page past the tile's last key is read as zeros (a row past the cache)
                int box_row = p.kv_rows;
                if (lane < 2 * HALVES) {
                    const int page_idx = (t.blk_lo + j) * 2 + pg_in_blk;
                    if (page_idx <= t.pos_last / PAGE) {
                        const int pg = p.block_table[(size_t)t.seq * p.table_stride + page_idx];
                        if (pg >= 0 && pg < p.n_pages) box_row = (pg * p.nkv + t.kvh) * PAGE;
                        else atomicOr(p.status, ESP_STATUS_BAD_INDEX);
                    }
                }
                if (lane == 0) {
                    ok = !*abort_flag && mbar_wait(&k_empty[s], ph ^ 1);
                    if (ok) mbar_expect_tx(&k_full[s], KV_BYTES);
                }
                ok = __shfl_sync(0xffffffffu, ok, 0);
                if (!ok) break;
                if (lane < 2 * HALVES)
                    tma_load_2d(k_s + s * KV_BYTES + half * ATOM_BYTES + pg_in_blk * (PAGE * 128), &map_k, half * 64, box_row, &k_full[s]);
                issued_k = g + 1;
                if (lane == 0) {
                    ok = !*abort_flag && mbar_wait(&v_empty[s], ph ^ 1);
                    if (ok) mbar_expect_tx(&v_full[s], KV_BYTES);
                }
                ok = __shfl_sync(0xffffffffu, ok, 0);
                if (!ok) break;
                if (lane < 2 * HALVES)
                    tma_load_2d(v_s + s * KV_BYTES + half * ATOM_BYTES + pg_in_blk * (PAGE * 128), &map_v, half * 64, box_row, &v_full[s]);
                issued_v = g + 1;
            }
        }
        if (lane == 0 && (!ok || *abort_flag)) {
            atomicOr(p.status, ESP_STATUS_WAIT_EXPIRED);
            *abort_flag = 1;
            // let this CTA's own copies land before its shared memory is given up
            if (issued_q > 0) mbar_wait(q_full, (issued_q - 1) & 1);
            for (int j = max(0, issued_k - STAGES); j < issued_k; j++) mbar_wait(&k_full[j % STAGES], (j / STAGES) & 1);
            for (int j = max(0, issued_v - STAGES); j < issued_v; j++) mbar_wait(&v_full[j % STAGES], (j / STAGES) & 1);
        }
    } else if (warp == 1) {
        if (lane == 0) {
            const unsigned idesc_s = idesc_attn(BN, false), idesc_pv = idesc_attn(HD, true);
            const unsigned long long dq = smem_desc(q_s), dk = smem_desc(k_s);
            const unsigned long long dv = smem_desc_mn(v_s, ATOM_BYTES);
            bool ok = true;
            int g = 0;
            auto issue_s = [&](int gg, bool last_of_item) {               // S = Q K^T of key block gg into S buffer gg % 2
                const int st = gg % STAGES;
                if (!mbar_wait(&k_full[st], (gg / STAGES) & 1)) return false;
                tc_fence_after();
#pragma unroll
                for (int kk = 0; kk < HD / 16; kk++) {
                    const unsigned off = ((kk >> 2) * ATOM_BYTES + (kk & 3) * 32) >> 4;
                    tc_mma(tm_s + (gg & 1) * BN, dq + off, dk + ((st * KV_BYTES) >> 4) + off, idesc_s, kk > 0 ? 1u : 0u);
                }
                tc_commit(&k_empty[st]);                                  // the keys are free once S is done
                if (last_of_item) tc_commit(q_empty);                     // and so are the queries after the item's last S
                tc_commit(&s_full[gg & 1]);
                return true;
            };
            for (int round = 0; ok && !*abort_flag; round++) {
                const int item = item_of(round);
                if (item >= n_items) break;
                const Item t = load_item(p, item);
                ok = mbar_wait(q_full, round & 1);
                if (ok) ok = issue_s(g, t.nb == 1);
                for (int j = 0; j < t.nb && ok && !*abort_flag; j++, g++) {
                    const int s = g & 1, st = g % STAGES;
                    if (j + 1 < t.nb) ok = issue_s(g + 1, j + 2 == t.nb);  // runs while the row threads work on this block
                    if (!ok) break;
                    // P stands where S of this block stood (and with that: PV of two blocks ago has been read),
                    // the values have landed.  S of the block after next goes to the same columns: the tensor
                    // core runs one thread's products in the order in which they were issued
                    if (!mbar_wait(p_ready, g & 1) || !mbar_wait(&v_full[st], (g / STAGES) & 1)) {
                        ok = false;
                        break;
                    }
                    tc_fence_after();
#pragma unroll
                    for (int kk = 0; kk < BN / 16; kk++) {
                        const unsigned b_off = (st * KV_BYTES + kk * 16 * 128) >> 4;
                        tc_mma_ta(tm_pv + s * BN, tm_s + s * BN + kk * 8, dv + b_off, idesc_pv, kk > 0 ? 1u : 0u);
                    }
                    tc_commit(&v_empty[st]);
                    tc_commit(&pv_full[s]);
                }
            }
            if (!ok) {
                atomicOr(p.status, ESP_STATUS_WAIT_EXPIRED);
                *abort_flag = 1;
            }
        }
    } else {
        // ---- row threads: TMEM lane = query row of the tile; ROWT threads a row.  The warps w, w + 4, w + 8 .. may
        // read the same 32 lanes; thread ``side`` of a row takes the keys side * CW .. of a block and the columns
        // side * OW .. of the head.  They exchange their maxima of a block through shared memory and meet at a
        // named barrier of their own (once when all have written, once when all have read); their sums stay
        // apart until the end.
        const int quad = warp & 3, r = quad * 32 + lane, side = (warp - 2) >> 2;
        const unsigned lane_sel = (unsigned)(quad * 32) << 16;
        const float sc = 1.4426950408889634f / sqrtf((float)HD);
        constexpr int CW = BN / ROWT;                                    // keys of a block that this thread takes
        constexpr int OW = HD / ROWT;                                    // columns of O that this thread keeps
        constexpr int MATES = ROWT * 32;                                 // threads at the row's named barrier
        static_assert(CW % 32 == 0 && OW % 32 == 0, "a thread reads TMEM 32 columns at a time");
        bool ok = true;
        int g = 0;
        for (int round = 0; ok; round++) {
            const int item = item_of(round);
            if (item >= n_items) break;
            const Item t = load_item(p, item);
            const int pos = t.pos0 + r;
            const int key_first = p.window > 0 ? pos - p.window + 1 : 0; // the keys this row sees: key_first .. pos
            float o[OW];
#pragma unroll
            for (int i = 0; i < OW; i++) o[i] = 0.f;
            float m_run = -INFINITY, l_run = 0.f, pending = 0.f;         // pending: the factor O takes before the last PV is added
            for (int j = 0; j < t.nb; j++, g++) {
                const int s = g & 1, key0 = (t.blk_lo + j) * BN;
                ok = !*abort_flag && mbar_wait(&s_full[s], (g >> 1) & 1);
                ok = pair_agree(ok, 1 + quad, MATES);                            // the two warps of a row go on or leave together
                if (!ok) break;
                tc_fence_after();
                // does any (row of the tile, key of the block) pair need the mask?
                const bool edge = key0 + BN - 1 > t.pos0 || (p.window > 0 && key0 < t.pos0 + BM - 1 - p.window + 1);
                // live columns of this row: c_lo .. c_lo + c_span; one unsigned comparison per element, no branch
                const int c_lo = key_first - key0 - side * CW;
                const unsigned c_span = (unsigned)(pos - key_first);
                const unsigned s_addr = tm_s + s * BN + lane_sel + side * CW;
                float mx = -INFINITY;                                     // of the raw scores: the scale is positive
                float sv[CW / 32][32];                                    // this thread's scores: read from TMEM once
#pragma unroll
                for (int c = 0; c < CW / 32; c++) {
                    tc_ld32(s_addr + c * 32, sv[c]);
                    if (edge) {
#pragma unroll
                        for (int i = 0; i < 32; i++) {
                            sv[c][i] = (unsigned)(c * 32 + i - c_lo) <= c_span ? sv[c][i] : -INFINITY;
                            mx = fmaxf(mx, sv[c][i]);
                        }
                    } else {
#pragma unroll
                        for (int i = 0; i < 32; i++) mx = fmaxf(mx, sv[c][i]);
                    }
                }
                xchg[side * 128 + r] = mx;
                named_sync(1 + quad, MATES);
#pragma unroll
                for (int o2 = 0; o2 < ROWT; o2++) mx = fmaxf(mx, xchg[o2 * 128 + r]);
                named_sync(1 + quad, MATES);                              // all have read: the next block may write
                mx *= sc;
                const float m_new = fmaxf(m_run, mx);
                const float m_use = m_new == -INFINITY ? 0.f : m_new;
                const float alpha = fast_exp2(m_run - m_use);             // m_run = -inf gives 0
                m_run = m_new;
                // every thread of the row holds its scores in registers by now, so P may go where S stood: the
                // weights of keys 2c and 2c + 1 of the block into column c of the S buffer
                float l_add = 0.f;
                unsigned packed[CW / 2];
#pragma unroll
                for (int c = 0; c < CW / 32; c++) {
#pragma unroll
                    for (int i = 0; i < 32; i += 2) {                     // a masked score is -inf: its weight is 0
                        const float p0 = fast_exp2(fmaf(sv[c][i], sc, -m_use)), p1 = fast_exp2(fmaf(sv[c][i + 1], sc, -m_use));
                        l_add += p0 + p1;
                        __nv_bfloat162 b = __floats2bfloat162_rn(p0, p1);
                        packed[c * 16 + (i >> 1)] = *reinterpret_cast<unsigned*>(&b);
                    }
                }
                const unsigned p_addr = tm_s + s * BN + lane_sel + side * (CW / 2);
                if constexpr (CW == 64) tc_st32(p_addr, packed);
                else tc_st16(p_addr, packed);
                tc_wait_st();
                l_run = l_run * alpha + l_add;
                tc_fence_before();                                        // S of this block has been read, P written
                __syncwarp();
                if (lane == 0) mbar_arrive(p_ready);
                if (j > 0) {                                              // O = O * factor + PV of the block before
                    ok = mbar_wait(&pv_full[s ^ 1], ((g - 1) >> 1) & 1);
                    ok = pair_agree(ok, 1 + quad, MATES);
                    if (!ok) break;
                    tc_fence_after();
#pragma unroll
                    for (int c = 0; c < OW / 32; c++) {
                        float v[32];
                        tc_ld32(tm_pv + (s ^ 1) * BN + lane_sel + side * OW + c * 32, v);
#pragma unroll
                        for (int i = 0; i < 32; i++) o[c * 32 + i] = o[c * 32 + i] * pending + v[i];
                    }
                }
                pending = alpha;
            }
            if (!ok) break;
            const int s = (g - 1) & 1;                                    // the item's last block
            ok = mbar_wait(&pv_full[s], ((g - 1) >> 1) & 1);
            ok = pair_agree(ok, 1 + quad, MATES);
            if (!ok) break;
            tc_fence_after();
#pragma unroll
            for (int c = 0; c < OW / 32; c++) {
                float v[32];
                tc_ld32(tm_pv + s * BN + lane_sel + side * OW + c * 32, v);
#pragma unroll
                for (int i = 0; i < 32; i++) o[c * 32 + i] = o[c * 32 + i] * pending + v[i];
            }
            tc_fence_before();
            xchg[side * 128 + r] = l_run;                                 // the sums of a row's threads
            named_sync(1 + quad, MATES);
            float l_all = 0.f;
#pragma unroll
            for (int o2 = 0; o2 < ROWT; o2++) l_all += xchg[o2 * 128 + r];  // keys in ascending order
            named_sync(1 + quad, MATES);
            if (r < t.rows) {
                const float inv = l_all > 0.f ? 1.0f / l_all : 0.f;
                bf16* orow = p.out + ((size_t)(t.row0 + r) * p.nh + t.h) * HD + side * OW;
#pragma unroll
                for (int i = 0; i < OW; i += 8) {
                    __nv_bfloat162 b0 = __floats2bfloat162_rn(o[i] * inv, o[i + 1] * inv);
                    __nv_bfloat162 b1 = __floats2bfloat162_rn(o[i + 2] * inv, o[i + 3] * inv);
                    __nv_bfloat162 b2 = __floats2bfloat162_rn(o[i + 4] * inv, o[i + 5] * inv);
                    __nv_bfloat162 b3 = __floats2bfloat162_rn(o[i + 6] * inv, o[i + 7] * inv);
                    *reinterpret_cast<uint4*>(orow + i) = make_uint4(*reinterpret_cast<unsigned*>(&b0), *reinterpret_cast<unsigned*>(&b1),
                                                                     *reinterpret_cast<unsigned*>(&b2), *reinterpret_cast<unsigned*>(&b3));
                }
            }
        }
        if (!ok && lane == 0) {
            atomicOr(p.status, ESP_STATUS_WAIT_EXPIRED);
            *abort_flag = 1;
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"(512));
    }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// a bfloat16 matrix [rows, cols] (row-major, contiguous) in boxes of box_rows x 64 columns, 128-byte swizzle, zeros outside
int make_map2d(CUtensorMap* map, const void* base, unsigned long long cols, unsigned long long rows, unsigned box_rows) {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) != cudaSuccess ||
            qres != cudaDriverEntryPointSuccess)
            return (int)cudaErrorNotSupported;
        fn = reinterpret_cast<EncodeTiledFn>(ptr);
    }
    const cuuint64_t dims[2] = {cols, rows};
    const cuuint64_t strides[1] = {cols * 2};
    const cuuint32_t box[2] = {64, box_rows};
    const cuuint32_t elem[2] = {1, 1};
    const CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : (int)cudaErrorInvalidValue;
}

template <int HD>
int launch(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv, const AttnParams& p, int n_tiles,
           cudaStream_t stream) {
    constexpr int ROWT = HD >= 128 ? 4 : 2;   // threads that share a query row
    // queries, STAGES blocks of keys and of values, barriers, the row threads' exchange; and 1024 bytes to round
    // the start up with, where the 227 KB of a block have room for them
    size_t smem = (size_t)(HD / 64) * ATOM_BYTES * (1 + 2 * STAGES) + 256 + ROWT * 128 * 4;
    if (smem + 1024 <= 232448) smem += 1024;
    static bool raised = false;
    if (!raised) {
        cudaError_t e = cudaFuncSetAttribute(attn_prefill_tc05_kernel<HD, ROWT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        raised = true;
    }
    static int sm_count = 0;
    if (!sm_count) {
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev);
        if (sm_count <= 0) sm_count = 148;
    }
    const long long items = (long long)n_tiles * p.nh;
    // with more items than SMs, blocks take pairs (a long item and a short one): as many blocks as halve the list
    long long grid = items <= sm_count ? items : (items + 1) / 2;
    if (grid > sm_count) grid = sm_count;
    AttnParams pp = p;
    pp.smem_bytes = (int)smem;
    attn_prefill_tc05_kernel<HD, ROWT><<<(int)grid, 64 + ROWT * 128, smem, stream>>>(mq, mk, mv, pp);
    return esp_launch_status();
}
}  // namespace

// q [n_tokens, nh, hd] and out the same shape, bfloat16; tile_seq / tile_first: the tiles of 128 new tokens
// (sequence, index of the tile's first token among the sequence's new tokens), best listed with the tiles
// that see the most keys first; hd 64 or 128; pages of 64 positions.
ESP_API int esp_attn_prefill_tc05(const void* q, long long n_tokens, const void* k_cache, const void* v_cache, void* out,
                                  const int* tile_seq, const int* tile_first, const int* seq_start, const int* seq_past,
                                  const int* block_table, int table_stride, int n_pages, int page, int n_tiles, int nh,
                                  int nkv, int hd, int window, int* status, cudaStream_t stream) {
    if (n_tiles <= 0) return 0;
    if (page != PAGE || (hd != 64 && hd != 128) || nkv <= 0 || nh % nkv != 0 || nh > 65535 || n_tokens <= 0)
        return (int)cudaErrorInvalidValue;
    const unsigned long long kv_rows = (unsigned long long)n_pages * nkv * PAGE;
    if (kv_rows >= (1ull << 31)) return (int)cudaErrorInvalidValue;
    CUtensorMap mq, mk, mv;
    int rc = make_map2d(&mq, q, (unsigned long long)nh * hd, (unsigned long long)n_tokens, BM);
    if (rc) return rc;
    rc = make_map2d(&mk, k_cache, (unsigned long long)hd, kv_rows, PAGE);
    if (rc) return rc;
    rc = make_map2d(&mv, v_cache, (unsigned long long)hd, kv_rows, PAGE);
    if (rc) return rc;
    AttnParams p{(bf16*)out, tile_seq, tile_first, seq_start, seq_past, block_table, table_stride, n_pages, nh, nkv,
                 window, (int)kv_rows, n_tiles, 0, status};
    if (hd == 64) return launch<64>(mq, mk, mv, p, n_tiles, stream);
    return launch<128>(mq, mk, mv, p, n_tiles, stream);
}
