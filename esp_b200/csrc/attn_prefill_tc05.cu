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
//   O += P V         tcgen05.mma, N = head size, K = 128 keys, accumulated in TMEM over the blocks of a group
//
// m is the row's running maximum, allowed to lag: O and the row's sum are rescaled (O in tensor memory, by
// the row's threads) only when the maximum has outgrown the one in use by more than 2^8, so most blocks
// need no pass over O at all.
//
// Warp 0 loads the queries and the keys, the last warp the values (TMA, page by page, into three-stage rings of
// their own: a load takes longer to land than a block of keys takes to work through, so two blocks have to be
// in flight; a key stage is free as soon as S is done), warp 1 issues the MMAs, the other warps are the row
// threads.  Two groups of them take the item's key blocks in turn (group 0 the even ones), each with a softmax
// of its own (maximum, sum, S and O in tensor memory: 4 x 128 = all 512 columns) that are merged at the item's
// end: while one group turns scores into weights, the tensor core works for the other.  Within a group, ROWT
// threads share a row (with one warp per scheduler the chain multiply, exp2, add, round would run at its
// latency).  Every wait is bounded.
//
// Measured on B200: about 800 TFLOP/s on long prompts, whatever the arrangement of the row threads (one, two
// or four to a row; one or two groups; two tiles of queries sharing each block of keys, which halves the
// traffic from L2): with 16 products of 128 x 128 x 16 to a block the thread that issues them is busy for
// most of a block's time.
//
// Head sizes 64 and 128.  The page size is 64.  Rows of the tile beyond the sequence's new tokens are
// computed and not stored; keys beyond a row's position are masked before the maximum is taken.
#include "tc05.cuh"

namespace {
using namespace tc05;
constexpr int BM = 128, BN = 128, PAGE = 64;   // warps: 0 queries and keys, 1 MMA, GROUPS * ROWT * 4 of row threads, values
constexpr int ATOM_BYTES = 128 * 128;           // 128 rows of 128 bytes: one 64-wide slice of a 128-row operand
constexpr int STAGES = 3;                       // blocks of keys (and of values) in shared memory
constexpr int GROUPS = 2;                       // groups of row threads: they take an item's key blocks in turn

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
// derives the same run of items, and the counters of key blocks (g), of items and of each group's blocks that
// choose the stage, the TMEM buffer and the phase of each mbarrier run on from one item to the next.
// ROWT: threads of a group that share a query row: each takes 128 / ROWT keys of a block and HD / ROWT columns of
// the group's O when it has to be rescaled.
template <int HD, int ROWT>
__global__ void __launch_bounds__(96 + GROUPS * ROWT * 128, 1)
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
    constexpr int N_BARS = 8 + 4 * STAGES;
    unsigned long long* q_full = bars;                    // [1]
    unsigned long long* q_empty = bars + 1;               // [1]
    unsigned long long* o_full = bars + 2;                // [1] every product of the item is done
    unsigned long long* o_free = bars + 3;                // [1] the row threads have read the item's O
    unsigned long long* s_full = bars + 4;                // [GROUPS]
    unsigned long long* p_ready = bars + 6;               // [GROUPS]
    unsigned long long* k_full = bars + 8;                // [STAGES]
    unsigned long long* k_empty = k_full + STAGES;        // [STAGES]
    unsigned long long* v_full = k_empty + STAGES;        // [STAGES]
    unsigned long long* v_empty = v_full + STAGES;        // [STAGES]
    unsigned* tmem_slot = reinterpret_cast<unsigned*>(bars + N_BARS);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    static_assert(N_BARS * 8 + 8 <= 256, "the barriers and the two words after them take 256 bytes");
    float* xchg = reinterpret_cast<float*>(bars) + 64;    // [GROUPS][ROWT][128]: maxima of a block; sums and maxima at the end
    // where shared memory is too short for the slack that rounding up to 1024 bytes needs, its start has to
    // be aligned already; the block refuses to run otherwise
    if (smem + Q_BYTES + 2 * STAGES * KV_BYTES + 256 + GROUPS * ROWT * 128 * 4 > smem_raw + p.smem_bytes) {
        if (threadIdx.x == 0) atomicOr(p.status, ESP_STATUS_SMEM_LAYOUT);
        return;
    }

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    constexpr int V_WARP = 2 + GROUPS * ROWT * 4;                        // warps: 0 keys, 1 MMA, row threads, values
    if (threadIdx.x == 0) {
        // o_free: one arrival per warp of row threads; p_ready: one per warp of the group; the others one
        for (int i = 0; i < N_BARS; i++) mbar_init(&bars[i], i == 3 ? GROUPS * ROWT * 4 : (i == 6 || i == 7) ? ROWT * 4 : 1);
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
    const unsigned tm_s = tmem_base, tm_o = tmem_base + 256;           // S of the groups at columns 0 and 128, O at 256 and 384

    if (warp == 0 || warp == V_WARP) {
        // ---- loads.  Warp 0: the queries (lanes 0..HALVES-1) and the keys; the last warp: the values.  Each works
        // through the same blocks of keys with a ring and barriers of its own, so neither waits for the other's
        // stages.  A lane's box: (page of the block, 64-column slice); the pages of 16 blocks are read from the
        // block table at once, one per lane, and handed out by shuffle.
        const bool is_k = warp == 0;
        unsigned char* ring = is_k ? k_s : v_s;
        unsigned long long* full = is_k ? k_full : v_full;
        unsigned long long* empty = is_k ? k_empty : v_empty;
        const CUtensorMap* map = is_k ? &map_k : &map_v;
        bool ok = true;
        const int pg_in_blk = lane / HALVES, half = lane % HALVES;      // lanes 0..2*HALVES-1 issue boxes
        int g = 0, issued_q = 0, issued = 0;
        for (int round = 0; ok; round++) {
            const int item = item_of(round);
            if (item >= n_items) break;
            const Item t = load_item(p, item);
            if (is_k) {
                if (lane == 0) {                                         // the last item's S products have read its queries
                    ok = !*abort_flag && mbar_wait(q_empty, (round & 1) ^ 1);
                    if (ok) mbar_expect_tx(q_full, Q_BYTES);
                }
                ok = __shfl_sync(0xffffffffu, ok, 0);
                if (!ok) break;
                if (lane < HALVES) tma_load_2d(q_s + lane * ATOM_BYTES, &map_q, t.h * HD + lane * 64, t.row0, q_full);
                issued_q = round + 1;
            }
            int rows16 = p.kv_rows;                                      // this lane's page of the 16 blocks at hand
            for (int j = 0; j < t.nb && ok; j++, g++) {
                const int s = g % STAGES, ph = (g / STAGES) & 1;
                if ((j & 15) == 0) {
                    // a page past the tile's last key is read as zeros (a row past the cache)
                    rows16 = p.kv_rows;
                    const int page_idx = (t.blk_lo + j) * 2 + lane;
                    if (page_idx <= t.pos_last / PAGE) {
                        const int pg = p.block_table[(size_t)t.seq * p.table_stride + page_idx];
                        if (pg >= 0 && pg < p.n_pages) rows16 = (pg * p.nkv + t.kvh) * PAGE;
                        else atomicOr(p.status, ESP_STATUS_BAD_INDEX);
                    }
                }
                const int box_row = __shfl_sync(0xffffffffu, rows16, ((j & 15) * 2 + pg_in_blk) & 31);
                if (lane == 0) {
                    ok = !*abort_flag && mbar_wait(&empty[s], ph ^ 1);
                    if (ok) mbar_expect_tx(&full[s], KV_BYTES);
                }
                ok = __shfl_sync(0xffffffffu, ok, 0);
                if (!ok) break;
                if (lane < 2 * HALVES)
                    tma_load_2d(ring + s * KV_BYTES + half * ATOM_BYTES + pg_in_blk * (PAGE * 128), map, half * 64, box_row, &full[s]);
                issued = g + 1;
            }
        }
        if (lane == 0 && (!ok || *abort_flag)) {
            atomicOr(p.status, ESP_STATUS_WAIT_EXPIRED);
            *abort_flag = 1;
            // let this warp's own copies land before the block's shared memory is given up
            if (issued_q > 0) mbar_wait(q_full, (issued_q - 1) & 1);
            for (int j = max(0, issued - STAGES); j < issued; j++) mbar_wait(&full[j % STAGES], (j / STAGES) & 1);
        }
    } else if (warp == 1) {
        if (lane == 0) {
            const unsigned idesc_s = idesc_attn(BN, false), idesc_pv = idesc_attn(HD, true);
            const unsigned long long dq = smem_desc(q_s), dk = smem_desc(k_s);
            const unsigned long long dv = smem_desc_mn(v_s, ATOM_BYTES);
            bool ok = true;
            int g0 = 0;                                                   // key blocks before this item
            int n_p0 = 0, n_p1 = 0;                                       // blocks of each group so far: the phase of p_ready
            for (int round = 0; ok && !*abort_flag; round++) {
                const int item = item_of(round);
                if (item >= n_items) break;
                const Item t = load_item(p, item);
                // S = Q K^T of the item's key block j, for the group j % 2, over where the group's last P stood: the
                // tensor core runs one thread's products in the order in which they were issued
                auto issue_s = [&](int j) {
                    const int gg = g0 + j, st = gg % STAGES, b = j & 1;
                    if (!mbar_wait(&k_full[st], (gg / STAGES) & 1)) return false;
                    tc_fence_after();
#pragma unroll
                    for (int kk = 0; kk < HD / 16; kk++) {
                        const unsigned off = ((kk >> 2) * ATOM_BYTES + (kk & 3) * 32) >> 4;
                        tc_mma(tm_s + b * BN, dq + off, dk + ((st * KV_BYTES) >> 4) + off, idesc_s, kk > 0 ? 1u : 0u);
                    }
                    tc_commit(&k_empty[st]);                              // the keys are free once S is done
                    if (j + 1 == t.nb) tc_commit(q_empty);                // and so are the queries after the item's last S
                    tc_commit(&s_full[b]);
                    return true;
                };
                ok = mbar_wait(q_full, round & 1);
                if (ok) ok = issue_s(0);
                if (ok && t.nb > 1) ok = issue_s(1);
                // the row threads have read the O of the item before
                if (ok) ok = mbar_wait(o_free, (round & 1) ^ 1);
                for (int j = 0; j < t.nb && ok && !*abort_flag; j++) {
                    const int gg = g0 + j, st = gg % STAGES, b = j & 1;
                    // the group's P stands where its S stood (and its O has been rescaled if it had to be), the
                    // values have landed
                    const int n_p = b ? n_p1 : n_p0;
                    if (!mbar_wait(&p_ready[b], n_p & 1) || !mbar_wait(&v_full[st], (gg / STAGES) & 1)) {
                        ok = false;
                        break;
                    }
                    if (b) n_p1++;
                    else n_p0++;
                    tc_fence_after();
#pragma unroll
                    for (int kk = 0; kk < BN / 16; kk++) {                // O of the group += P V; its first block starts it
                        const unsigned b_off = (st * KV_BYTES + kk * 16 * 128) >> 4;
                        tc_mma_ta(tm_o + b * BN, tm_s + b * BN + kk * 8, dv + b_off, idesc_pv, (j >= GROUPS || kk > 0) ? 1u : 0u);
                    }
                    tc_commit(&v_empty[st]);
                    if (j + 1 == t.nb) tc_commit(o_full);                 // all of the item's products
                    if (j + GROUPS < t.nb) ok = issue_s(j + GROUPS);      // the group's next block
                }
                g0 += t.nb;
            }
            if (!ok) {
                atomicOr(p.status, ESP_STATUS_WAIT_EXPIRED);
                *abort_flag = 1;
            }
        }
    } else {
        // ---- row threads: TMEM lane = query row of the tile.  Two groups take the item's key blocks in turn (group
        // 0 the even ones), each with a softmax of its own (maximum, sum, O in tensor memory) that are merged at the
        // item's end: while one group turns its scores into weights, the other reads, compares and waits, so the
        // special function unit and the tensor core both stay busy.  ROWT threads of a group share a row: thread
        // ``side`` takes the keys side * CW .. of a block; they exchange their maxima through shared memory and
        // meet at a named barrier of their own (once when all have written, once when all have read).
        const int quad = warp & 3, r = quad * 32 + lane, grp = (warp - 2) / (4 * ROWT), side = ((warp - 2) >> 2) % ROWT;
        const unsigned lane_sel = (unsigned)(quad * 32) << 16;
        const float sc = 1.4426950408889634f / sqrtf((float)HD);
        constexpr int CW = BN / ROWT;                                    // keys of a block that this thread takes
        constexpr int OW = HD / ROWT;                                    // columns of the group's O that this thread rescales
        constexpr int FW = HD / (GROUPS * ROWT);                         // columns of the result that this thread writes
        constexpr int MATES = ROWT * 32, ROW_ALL = GROUPS * ROWT * 32;   // threads at the group's and at the row's barrier
        constexpr float LAZY = 8.f;                                      // O is rescaled when the maximum grew by more (log2)
        static_assert(CW % 32 == 0, "a thread reads its scores 32 columns at a time");
        static_assert(OW % 32 == 0 && (FW == 16 || FW == 32), "columns are read 32 or 16 at a time");
        const int bar_grp = 1 + grp * 4 + quad, bar_row = 1 + GROUPS * 4 + quad;
        float* xg = xchg + grp * (ROWT * 128);                            // the group's [side][row]
        bool ok = true;
        int n_b = 0;                                                      // blocks of this group so far
        for (int round = 0; ok; round++) {
            const int item = item_of(round);
            if (item >= n_items) break;
            const Item t = load_item(p, item);
            const int pos = t.pos0 + r;
            const int key_first = p.window > 0 ? pos - p.window + 1 : 0; // the keys this row sees: key_first .. pos
            float m_ref = -INFINITY, l_run = 0.f;                         // the maximum that O and l_run are scaled by
            for (int j = grp; j < t.nb && ok; j += GROUPS, n_b++) {
                const int key0 = (t.blk_lo + j) * BN;
                ok = !*abort_flag && mbar_wait(&s_full[grp], n_b & 1);
                ok = pair_agree(ok, bar_grp, MATES);                      // the threads of a row go on or leave together
                if (!ok) break;
                // S is done, and so are the products issued before it: the group's O holds its blocks so far
                tc_fence_after();
                // does any (row of the tile, key of the block) pair need the mask?
                const bool edge = key0 + BN - 1 > t.pos0 || (p.window > 0 && key0 < t.pos0 + BM - 1 - p.window + 1);
                // live columns of this row: c_lo .. c_lo + c_span; one unsigned comparison per element, no branch
                const int c_lo = key_first - key0 - side * CW;
                const unsigned c_span = (unsigned)(pos - key_first);
                const unsigned s_addr = tm_s + grp * BN + lane_sel + side * CW;
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
                xg[side * 128 + r] = mx;
                named_sync(bar_grp, MATES);
#pragma unroll
                for (int o2 = 0; o2 < ROWT; o2++) mx = fmaxf(mx, xg[o2 * 128 + r]);
                named_sync(bar_grp, MATES);                               // all have read: the next block may write
                const float m_new = fmaxf(m_ref, mx * sc);
                // The weights are exp2(score - m_ref) with a maximum that may lag behind by up to LAZY: they stay
                // below 2^LAZY, and sum and O stay consistent.  A row that outgrows that is brought up to date:
                // the sum here, O in tensor memory, which the warp reads and writes as a whole (the other rows
                // take the factor 1, so no row's result depends on its neighbours).  The group's first block has
                // nothing to rescale.
                const bool grew = m_new > m_ref + LAZY;                   // the same for all threads of the row
                if (j < GROUPS) {
                    m_ref = m_new;
                } else if (__any_sync(0xffffffffu, grew)) {
                    const float alpha = grew ? fast_exp2(m_ref - m_new) : 1.f;   // m_ref = -inf gives 0
                    if (grew) m_ref = m_new;
                    l_run *= alpha;
#pragma unroll
                    for (int c = 0; c < OW / 16; c++) {                   // in small pieces: the scores stay in registers
                        const unsigned o_addr = tm_o + grp * BN + lane_sel + side * OW + c * 16;
                        float v[16];
                        unsigned w[16];
                        tc_ld16(o_addr, v);
#pragma unroll
                        for (int i = 0; i < 16; i++) w[i] = __float_as_uint(v[i] * alpha);
                        tc_st16(o_addr, w);
                    }
                }
                const float m_use = m_ref == -INFINITY ? 0.f : m_ref;
                // every thread of the row holds its scores in registers by now, so P may go where S stood: the
                // weights of keys 2c and 2c + 1 of the block into column c of the group's S buffer
                float l_add = 0.f;
                const unsigned p_addr = tm_s + grp * BN + lane_sel + side * (CW / 2);
#pragma unroll
                for (int c = 0; c < CW / 32; c++) {
                    unsigned packed[16];
#pragma unroll
                    for (int i = 0; i < 32; i += 2) {                     // a masked score is -inf: its weight is 0
                        const float p0 = fast_exp2(fmaf(sv[c][i], sc, -m_use)), p1 = fast_exp2(fmaf(sv[c][i + 1], sc, -m_use));
                        l_add += p0 + p1;
                        __nv_bfloat162 b2 = __floats2bfloat162_rn(p0, p1);
                        packed[i >> 1] = *reinterpret_cast<unsigned*>(&b2);
                    }
                    tc_st16(p_addr + c * 16, packed);
                }
                tc_wait_st();
                l_run += l_add;
                tc_fence_before();                                        // S has been read, P and O written
                __syncwarp();
                if (lane == 0) mbar_arrive(&p_ready[grp]);
            }
            // ---- the item's end: the sum of the group's threads, then (sum, maximum) of every group to all the
            // row's threads, who wait for the last products and each write HD / (GROUPS * ROWT) columns
            xg[side * 128 + r] = l_run;
            named_sync(bar_grp, MATES);
            float l_grp = 0.f;
#pragma unroll
            for (int o2 = 0; o2 < ROWT; o2++) l_grp += xg[o2 * 128 + r];  // keys in ascending order
            named_sync(bar_grp, MATES);
            if (side == 0) xg[r] = l_grp;
            if (side == 1) xg[128 + r] = m_ref;
            if (ok) ok = !*abort_flag && mbar_wait(o_full, round & 1);
            ok = pair_agree(ok, bar_row, ROW_ALL);                        // all threads of the row: written, and well
            if (!ok) break;
            tc_fence_after();
            float m_all = -INFINITY, f[GROUPS], l_all = 0.f;
#pragma unroll
            for (int b = 0; b < GROUPS; b++) m_all = fmaxf(m_all, xchg[b * (ROWT * 128) + 128 + r]);
#pragma unroll
            for (int b = 0; b < GROUPS; b++) {                            // a group without a key for this row counts 0
                const float m_b = xchg[b * (ROWT * 128) + 128 + r];
                f[b] = m_b == -INFINITY ? 0.f : fast_exp2(m_b - m_all);
                l_all += f[b] * xchg[b * (ROWT * 128) + r];
            }
            const float inv = l_all > 0.f ? 1.0f / l_all : 0.f;
            const int col0 = (grp * ROWT + side) * FW;
            float o[FW];
#pragma unroll
            for (int i = 0; i < FW; i++) o[i] = 0.f;
#pragma unroll
            for (int b = 0; b < GROUPS; b++) {
                if (b < t.nb) {                                           // an item of one block has nothing from the second group
                    float v[FW];
                    if constexpr (FW == 32) tc_ld32(tm_o + b * BN + lane_sel + col0, v);
                    else tc_ld16(tm_o + b * BN + lane_sel + col0, v);
#pragma unroll
                    for (int i = 0; i < FW; i++) o[i] += f[b] * v[i];
                }
            }
            tc_fence_before();
            named_sync(bar_row, ROW_ALL);                                 // all have read the sums: the next item may write
            if (lane == 0) mbar_arrive(o_free);
            if (r < t.rows) {
                bf16* orow = p.out + ((size_t)(t.row0 + r) * p.nh + t.h) * HD + col0;
#pragma unroll
                for (int i = 0; i < FW; i += 8) {
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
    constexpr int ROWT = 2;      // threads of a group that share a query row
    // queries, STAGES blocks of keys and of values, barriers, the row threads' exchange; and 1024 bytes to round
    // the start up with, where the 227 KB of a block have room for them
    size_t smem = (size_t)(HD / 64) * ATOM_BYTES * (1 + 2 * STAGES) + 256 + GROUPS * ROWT * 128 * 4;
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
    // one block per SM; with more items than that, the blocks that got the shortest items take a second one
    const long long grid = items < sm_count ? items : sm_count;
    AttnParams pp = p;
    pp.smem_bytes = (int)smem;
    attn_prefill_tc05_kernel<HD, ROWT><<<(int)grid, 96 + GROUPS * ROWT * 128, smem, stream>>>(mq, mk, mv, pp);
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
