// Tensor-core matrix product for many rows (prefill) on the 5th-generation
// tensor cores: operands travel global -> shared memory by TMA
// (cp.async.bulk.tensor, 128-byte swizzle), tcgen05.mma accumulates in tensor
// memory (TMEM), and the epilogue reads the accumulator back with tcgen05.ld.
//
//   PLAIN:  C[m, n]   = scale[m] * sum_k A[m, k] * W[g][n, k]                (float out)
//   SWIGLU: act[m, j] = silu(A W_gate[g][j]) * (A W_up[g][j])                (bfloat16 out)
//           W[g] = [gate rows; up rows]
//
// A is [rows, K] bfloat16, rows sorted by group; W is [G, Nw, K] bfloat16 (G = 1
// for a dense product).  The weights are the 128-row operand of the MMA and a
// run of up to 128 or 256 token rows is its N side, so the accumulator holds
// D[feature, token]: TMEM lane = output feature, TMEM column = token.  The width
// of a token tile is whatever its group has left, rounded up to 16, which keeps
// ragged groups (a handful of rows for one expert, hundreds for another) from
// wasting tensor work.  A token tile never mixes groups: the tile list (group,
// first row, rows) is made on the device by the routing kernels.
//
// One tile = 128 weight rows x one token tile.  PLAIN: the rows are 128 output
// features.  SWIGLU: they are the gate rows of 64 features followed by the up rows
// of the same 64 features, so that one MMA per 16-wide k step makes both and one
// accumulator of n_tok columns holds them (lanes 0..63 gate, 64..127 up).  A
// tcgen05.mma with M = 128 keeps its issuing thread for about 83 cycles at any
// N up to 128 and for 128 cycles at N = 256 (measured), so few wide MMAs beat many
// narrow ones: token tiles reach 256 rows.  Warps 0 and 6 issue the TMA loads (the
// k steps in turn, each into a ring of its own), warp 1 owns TMEM and issues the
// MMAs, warps 2..5 and 7..10 are the epilogue (each reads the 32 TMEM lanes that its
// position in the warpgroup may touch; the two sets take alternate runs of 32 tokens).  The
// rings' stages are handed back and forth with mbarriers.  Every wait is
// bounded: if one runs out the kernel raises ESP_STATUS_WAIT_EXPIRED in the
// status word, stops issuing work, lets its own copies land, frees its TMEM and
// returns.
#include <type_traits>

#include "tc05.cuh"

namespace {
using namespace tc05;
constexpr int BF = 128;            // features (weight rows) per tile: the M side of the MMA
constexpr int TOK_BOX = 16;         // token rows per TMA box; a tile's width is a multiple of it
constexpr int BK = 64, THREADS = 352;   // warps: 0 producer, 1 MMA, 2..5 epilogue, 6 producer, 7..10 epilogue
constexpr int W_BYTES = BF * BK * 2;

struct Tc05Params {
    const int* tile_group;        // [tiles] or null (dense)
    const int* tile_row0;         // [tiles]
    const int* tile_rows;         // [tiles]
    const int* n_tiles;           // device scalar or null
    const float* row_scale;       // [rows] or null
    void* C;
    long long ldc;
    int M, N, K;                  // N: output columns (SWIGLU: the intermediate size)
    int* status;
};

// Instruction descriptor: bfloat16 x bfloat16 -> float, both operands K-major, M = 128, N = n.
__device__ __forceinline__ unsigned instr_desc(int n, int m = BF) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((unsigned)(n >> 3) << 17) | ((unsigned)(m >> 4) << 24);
}

// Persistent form: a CTA per SM walks the list of (token tile, feature tile) pairs with stride gridDim.x.
// The producer runs ahead across tile boundaries, so the weight stream never pauses; the accumulator is
// double-buffered in TMEM, so the epilogue of one tile overlaps the MMAs of the next.
//
// Each producer warp has a ring of its own, and a ring is a byte queue: a stage takes the 16 KB of its
// weight rows and 128 bytes for each of its tile's token rows, not the room of the widest tile, so that
// short tiles keep more k steps in flight (a load takes a microsecond or more to arrive).  A stage that
// would run over the end of its ring starts at the front again and owns the bytes it skipped.  The
// producer and the MMA thread derive the same offsets from the same list of tiles.
//
// What bounds a k step is the time its instructions keep the issuing threads (measured here: a wait on an
// mbarrier that is already complete 185 cycles, expect_tx 50, the first cp.async.bulk.tensor of a thread
// 310 and each further one 145, or 50 when other lanes of the warp issue them in the same instruction; a
// tcgen05.mma 83).  So the loads of a stage are issued by several lanes at once, and two producer warps
// take the k steps in turn.
constexpr int PRODUCERS = 2;               // warps that issue the loads, taking the k steps in turn
constexpr int RING_KB = 96, RING_BYTES = RING_KB * 1024;    // each producer's own ring
// GROUP consecutive k steps (one of each ring) share a pair of mbarriers: one wait before their MMAs, one commit
// after them.  A wait on a complete barrier and a commit keep the MMA thread about 100 cycles each, as long as
// two of a k step's four MMAs, and that thread's time is what a k step takes (measured with clock64: the
// copies are there long before, the producers wait for room).  Wider groups were measured and lose: four k steps
// behind one wait and one commit, or behind one wait with a commit for every two (2,048 tokens, 24 layers: 15.1
// and 13.7 ms against 12.7), because the rings then hold too few groups for the copies to run ahead.
constexpr int GROUP = 2;
constexpr int NSLOT = 8;                   // groups of stages in flight at most (pairs of mbarriers)
constexpr int BAR_BYTES = 512;             // the mbarriers and two words behind the ring
constexpr int SWAP_BYTES = 2 * 2 * 2 * 2 * 16 * 32 * 4;   // the epilogue's exchange of gate and up halves

struct TileInfo {
    int group, row0, n_rows, n_tok, f0;
};

// PAIR: two CTAs of a cluster work on one token tile and two neighbouring feature tiles (rank 0 the even one):
// ``feat_tiles`` then counts pairs of feature tiles, and the tile's width is a multiple of 32 so that each CTA
// loads a half that is whole boxes.
template <int MAX_TOK, int FEATS, bool PAIR>
__device__ __forceinline__ TileInfo tile_info(const Tc05Params& p, int tile, int feat_tiles, int rank) {
    TileInfo t;
    const int tt = tile / feat_tiles;
    const int ft = PAIR ? 2 * (tile - tt * feat_tiles) + rank : tile - tt * feat_tiles;   // feature tiles vary fastest: neighbours share tokens
    if (p.tile_group) {
        t.group = p.tile_group[tt];
        t.row0 = p.tile_row0[tt];
        t.n_rows = min(MAX_TOK, p.tile_rows[tt]);
    } else {
        t.group = 0;
        t.row0 = tt * MAX_TOK;
        t.n_rows = min(MAX_TOK, p.M - t.row0);
    }
    constexpr int STEP = PAIR ? 2 * TOK_BOX : TOK_BOX;
    t.n_tok = min(MAX_TOK, (max(t.n_rows, 1) + STEP - 1) / STEP * STEP);
    t.f0 = ft * FEATS;
    return t;
}

// ---- what a pair of CTAs needs (cta_group::2): one thread of the leader (rank 0) issues MMAs of 256 rows, the
// upper 128 being the peer's weight rows; each CTA holds half of the token rows; copies of both CTAs count
// on the leader's barriers; the leader's commits reach the barriers of both.
__device__ __forceinline__ unsigned cluster_rank() {
    unsigned r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;\n" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;\n" ::: "memory");
}
// the copy lands in this CTA's shared memory; its bytes are counted on the barrier at the same place in the
// pair's first CTA (bit 24 of a shared::cluster address tells the two CTAs of a pair apart)
__device__ __forceinline__ void tma_load_3d_pair(void* dst, const CUtensorMap* map, int c0, int c1, int c2, void* bar) {
    asm volatile(
        "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];\n"
        ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar) & 0xFEFFFFFFu), "r"(c0), "r"(c1), "r"(c2) : "memory");
}
__device__ __forceinline__ void tc_mma_lo_pair(unsigned tmem_d, unsigned a_lo, unsigned b_lo, unsigned hi, unsigned idesc,
                                               unsigned accumulate) {
    asm volatile(
        "{\n.reg .pred p;\n.reg .b64 da, db;\n"
        "setp.ne.b32 p, %5, 0;\n"
        "mov.b64 da, {%1, %3};\n"
        "mov.b64 db, {%2, %3};\n"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], da, db, %4, p;\n}\n"
        ::"r"(tmem_d), "r"(a_lo), "r"(b_lo), "r"(hi), "r"(idesc), "r"(accumulate) : "memory");
}
// the barrier at this address in both CTAs of the pair gets an arrival once the MMAs issued so far are done
__device__ __forceinline__ void tc_commit_pair_addr(unsigned bar_addr) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;\n"
                 ::"r"(bar_addr), "h"((unsigned short)3) : "memory");
}
// an arrival on the barrier at this address in the pair's first CTA
__device__ __forceinline__ void mbar_arrive_leader(void* bar) {
    unsigned remote;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;\n" : "=r"(remote) : "r"(smem_u32(bar)), "r"(0));
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];\n" ::"r"(remote) : "memory");
}

// MAX_TOK: token rows per tile at most (the N side of the MMA): 128 or 256.  Two accumulators of MAX_TOK
// columns fit the 512 columns of TMEM in either case.
template <bool SWIGLU, int MAX_TOK, bool PAIR>
__global__ void __launch_bounds__(THREADS, 1)
gemm_tc05_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_a64,
                 const __grid_constant__ CUtensorMap map_a128, const __grid_constant__ CUtensorMap map_w, Tc05Params p) {
    constexpr int TOK_BYTES = MAX_TOK * BK * 2;
    static_assert(2 * (W_BYTES + TOK_BYTES) <= RING_BYTES, "two stages of the widest tile must fit a ring");
    constexpr int FEATS = SWIGLU ? BF / 2 : BF;                  // output features of one tile
    constexpr int ACC_COLS = MAX_TOK;                            // TMEM columns of one accumulator buffer
    constexpr int NBUF = 2;
    constexpr int TMEM_COLS = NBUF * ACC_COLS;
    static_assert(TMEM_COLS <= 512, "the accumulators do not fit");
    static_assert(GROUP == PRODUCERS, "a ring holds one stage of a group, which fits whatever was skipped at the ring's end");
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    unsigned long long* full_bar = reinterpret_cast<unsigned long long*>(smem + PRODUCERS * RING_BYTES);   // [slot]
    unsigned long long* empty_bar = full_bar + NSLOT;
    unsigned long long* acc_full_bar = empty_bar + NSLOT;            // [2]
    unsigned long long* acc_empty_bar = acc_full_bar + 2;        // [2]
    unsigned* tmem_slot = reinterpret_cast<unsigned*>(acc_empty_bar + 2);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    float* swap = reinterpret_cast<float*>(smem + PRODUCERS * RING_BYTES + BAR_BYTES);     // SWIGLU: [2 halves][2][2 pairs][2 roles][16][32]

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int rank = PAIR ? (int)cluster_rank() : 0;                 // this CTA within its pair
    const int unit = PAIR ? blockIdx.x >> 1 : blockIdx.x;            // the CTA (or pair) among those of the grid
    const int n_units = PAIR ? gridDim.x >> 1 : gridDim.x;
    const int feat_tiles = PAIR ? ((p.N + FEATS - 1) / FEATS + 1) / 2 : (p.N + FEATS - 1) / FEATS;
    const int token_tiles = p.tile_group ? *p.n_tiles : (p.M + MAX_TOK - 1) / MAX_TOK;
    const int total_tiles = token_tiles * feat_tiles;
    if (unit >= total_tiles) return;                                 // the whole CTA (pair) leaves before any barrier exists
    const int k_iters = (p.K + BK - 1) / BK;

    if (threadIdx.x == 0) {
        for (int s = 0; s < NSLOT; s++) {
            mbar_init(&full_bar[s], GROUP);                          // one announcement per k step of the group
            mbar_init(&empty_bar[s], 1);
        }
        for (int b = 0; b < 2; b++) {
            mbar_init(&acc_full_bar[b], 1);
            mbar_init(&acc_empty_bar[b], PAIR ? 16 : 8);             // one arrival per epilogue warp (of both CTAs)
        }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    if (warp == 1) {
        if (PAIR) {
            asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_u32(tmem_slot)), "r"(TMEM_COLS));
            asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;\n" ::);
        } else {
            asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_u32(tmem_slot)), "r"(TMEM_COLS));
            asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::);
        }
    }
    tc_fence_before();
    __syncthreads();
    if (PAIR) cluster_sync_all();                                    // the peer's barriers exist before anything reaches them
    tc_fence_after();
    const unsigned tmem_base = *tmem_slot;

    if (warp == 0 || warp == 6) {
        // Producer warps: warp 0 takes the even k steps of the CTA's run of tiles, warp 6 the odd ones.  Lane 0
        // waits for the stage and announces its bytes; then the lanes issue one box each in one instruction:
        // lane 0 the weight rows (PLAIN: 128 rows; SWIGLU: the 64 gate rows), lane 1 the 64 up rows, lanes 2..
        // the token rows in boxes of 128, then 64, then 16.
        const int me = warp == 0 ? 0 : 1;
        unsigned char* ring = smem + me * RING_BYTES;
        int it = 0;                                                  // k steps of the CTA so far
        int tail = 0;                                                // the oldest group whose bytes in this ring are not yet known free
        int off_kb = 0, free_kb = RING_KB;
        unsigned long long held = 0;                                 // lane 0: KB that this ring holds for each group in flight, 8 bits a slot
        bool ok = true;
        // lane 0, before a k step's copies: the step's group has a slot (the group NSLOT before it was consumed)
        // and the ring has room; the bytes of consumed groups come back as their barriers complete
        auto acquire = [&](int grp, int need_kb) {
            ok = !*abort_flag;
            while (ok && (free_kb < need_kb || grp - tail >= NSLOT)) {
                if (tail >= grp) {                                    // nothing older is left to come back: never wait on the step's own group
                    ok = false;
                    break;
                }
                ok = mbar_wait(&empty_bar[tail % NSLOT], (tail / NSLOT) & 1);
                free_kb += (int)((held >> (8 * (tail % NSLOT))) & 0xFF);
                held &= ~(0xFFull << (8 * (tail % NSLOT)));
                tail++;
            }
            held += (unsigned long long)need_kb << (8 * (grp % NSLOT));
            free_kb -= need_kb;
        };
        TileInfo next = tile_info<MAX_TOK, FEATS, PAIR>(p, unit, feat_tiles, rank);
        for (int tile = unit; tile < total_tiles && ok; tile += n_units) {
            const TileInfo t = next;
            if (tile + n_units < total_tiles)                         // the list entry of the next tile is fetched early
                next = tile_info<MAX_TOK, FEATS, PAIR>(p, tile + n_units, feat_tiles, rank);
            // token rows that this CTA loads: all of the tile, or its half of a pair's tile
            const int my_tok = PAIR ? t.n_tok >> 1 : t.n_tok, tok0 = PAIR ? rank * my_tok : 0;
            const unsigned my_tx = W_BYTES + my_tok * BK * 2;
            const unsigned stage_tx = PAIR ? 2 * my_tx : my_tx;       // what the (leader's) barrier is told to expect
            const int size_kb = my_tx >> 10;                          // my_tok is a multiple of 16: whole KB
            // this lane's box: the map, the row it starts at, the bytes into the stage
            const int n128 = my_tok >> 7, n64 = (my_tok >> 6) & 1, n16 = (my_tok >> 4) & 3;
            const CUtensorMap* box_map = nullptr;
            int box_row = 0, box_grp = 0, box_off = 0;
            if (lane == 0) {
                box_map = &map_w, box_row = t.f0, box_grp = t.group;
            } else if (lane == 1) {
                if (SWIGLU) box_map = &map_w, box_row = p.N + t.f0, box_grp = t.group, box_off = W_BYTES / 2;
            } else {
                const int j = lane - 2;
                int r = -1;
                if (j < n128) r = j * 128, box_map = &map_a128;
                else if (j < n128 + n64) r = n128 * 128, box_map = &map_a64;
                else if (j < n128 + n64 + n16) r = n128 * 128 + n64 * 64 + (j - n128 - n64) * TOK_BOX, box_map = &map_a;
                if (r >= 0) box_row = t.row0 + tok0 + r, box_off = W_BYTES + r * BK * 2;
            }
            for (int k = 0; k < k_iters && ok; k++, it++) {
                if (it % PRODUCERS != me) continue;
                const bool wrap = off_kb + size_kb > RING_KB;
                const int need_kb = size_kb + (wrap ? RING_KB - off_kb : 0);
                const int s = (it / GROUP) % NSLOT;
                if (lane == 0) {
                    acquire(it / GROUP, need_kb);
                    if (ok && rank == 0) mbar_expect_tx(&full_bar[s], stage_tx);
                }
                ok = __shfl_sync(0xffffffffu, ok, 0);
                if (!ok) break;
                if (wrap) off_kb = 0;
                if (box_map) {
                    if (PAIR) tma_load_3d_pair(ring + off_kb * 1024 + box_off, box_map, k * BK, box_row, box_grp, &full_bar[s]);
                    else tma_load_3d(ring + off_kb * 1024 + box_off, box_map, k * BK, box_row, box_grp, &full_bar[s]);
                }
                off_kb += size_kb;
            }
        }
        // the CTA's last group may be short of k steps: the barrier still wants an announcement for each
        for (const int end = (it + GROUP - 1) / GROUP * GROUP; it < end && ok; it++) {
            if (it % PRODUCERS != me) continue;
            if (lane == 0) {
                acquire(it / GROUP, 0);
                if (ok && rank == 0) mbar_arrive(&full_bar[(it / GROUP) % NSLOT]);
            }
            ok = __shfl_sync(0xffffffffu, ok, 0);
        }
        if (lane == 0 && (!ok || *abort_flag)) {
            atomicOr(p.status, ESP_STATUS_WAIT_EXPIRED);
            *abort_flag = 1;
            // let this warp's own copies land before the CTA's shared memory is given up: a millisecond, far more
            // than a copy takes (their barriers also count the other producer's copies, which may never come)
            for (int j = 0; j < 1000; j++) __nanosleep(1000);
        }
    } else if (warp == 1) {
        if (lane == 0 && rank == 0) {                                // of a pair, the first CTA issues the MMAs of both
            int local = 0;
            int off0 = 0, off1 = 0;                                   // per ring: the next offset (KB)
            int step = 0;                                             // k steps of the CTA so far
            const int my_steps = ((total_tiles - unit + n_units - 1) / n_units) * k_iters;
            // descriptors differ from stage to stage and from one 16-wide k step to the next only in the
            // address field (16-byte units): the low word is a base plus a constant
            const unsigned long long desc0 = smem_desc(smem);
            const unsigned desc_hi = (unsigned)(desc0 >> 32), desc_lo0 = (unsigned)desc0;
            const unsigned full_addr = smem_u32(full_bar), empty_addr = smem_u32(empty_bar);
            bool ok = true;
            // One k step out of ring R: four MMAs.  The first k step of a group waits for the group's copies (of
            // both rings), the last one hands the group's stages back: a wait and a commit keep this thread about
            // 100 cycles each, as long as two MMAs, and this thread's time is what a k step takes.
            auto k_step = [&](auto ring_tag, int& off, unsigned acc, unsigned idesc, int size_kb, bool first) {
                constexpr int R = decltype(ring_tag)::value;
                const int grp = step / GROUP, in_grp = step - grp * GROUP;
                const unsigned slot8 = (unsigned)(grp & (NSLOT - 1)) << 3;
                if (in_grp == 0) {
                    if (!mbar_wait_addr(full_addr + slot8, (grp >> 3) & 1)) return false;
                    tc_fence_after();
                }
                if (off + size_kb > RING_KB) off = 0;                   // the producer's rule
                const unsigned w_lo = desc_lo0 + (R * RING_KB + off) * (1024 >> 4);
                const unsigned t_lo = w_lo + (W_BYTES >> 4);
                off += size_kb;
                step++;
                const bool last = in_grp == GROUP - 1 || step == my_steps;
                if (PAIR) {
                    tc_mma_lo_pair(acc, w_lo, t_lo, desc_hi, idesc, first ? 0u : 1u);
                    tc_mma_lo_pair(acc, w_lo + 2, t_lo + 2, desc_hi, idesc, 1u);
                    tc_mma_lo_pair(acc, w_lo + 4, t_lo + 4, desc_hi, idesc, 1u);
                    tc_mma_lo_pair(acc, w_lo + 6, t_lo + 6, desc_hi, idesc, 1u);
                    if (last) tc_commit_pair_addr(empty_addr + slot8);  // the stages are free in both CTAs once these MMAs have read them
                } else {
                    tc_mma_lo(acc, w_lo, t_lo, desc_hi, idesc, first ? 0u : 1u);
                    tc_mma_lo(acc, w_lo + 2, t_lo + 2, desc_hi, idesc, 1u);
                    tc_mma_lo(acc, w_lo + 4, t_lo + 4, desc_hi, idesc, 1u);
                    tc_mma_lo(acc, w_lo + 6, t_lo + 6, desc_hi, idesc, 1u);
                    if (last) tc_commit_addr(empty_addr + slot8);       // the stages are free once these MMAs have read them
                }
                return true;
            };
            // a whole group in one piece: the two k steps of a tile that lie in one group, without a branch between them
            auto two_steps = [&](unsigned acc, unsigned idesc, int size_kb, bool first) {
                const int grp = step / GROUP;
                const unsigned slot8 = (unsigned)(grp & (NSLOT - 1)) << 3;
                if (!mbar_wait_addr(full_addr + slot8, (grp >> 3) & 1)) return false;
                tc_fence_after();
                if (off0 + size_kb > RING_KB) off0 = 0;
                if (off1 + size_kb > RING_KB) off1 = 0;
                const unsigned w0 = desc_lo0 + off0 * (1024 >> 4), t0 = w0 + (W_BYTES >> 4);
                const unsigned w1 = desc_lo0 + (RING_KB + off1) * (1024 >> 4), t1 = w1 + (W_BYTES >> 4);
                off0 += size_kb;
                off1 += size_kb;
                step += 2;
                if (PAIR) {
                    tc_mma_lo_pair(acc, w0, t0, desc_hi, idesc, first ? 0u : 1u);
                    tc_mma_lo_pair(acc, w0 + 2, t0 + 2, desc_hi, idesc, 1u);
                    tc_mma_lo_pair(acc, w0 + 4, t0 + 4, desc_hi, idesc, 1u);
                    tc_mma_lo_pair(acc, w0 + 6, t0 + 6, desc_hi, idesc, 1u);
                    tc_mma_lo_pair(acc, w1, t1, desc_hi, idesc, 1u);
                    tc_mma_lo_pair(acc, w1 + 2, t1 + 2, desc_hi, idesc, 1u);
                    tc_mma_lo_pair(acc, w1 + 4, t1 + 4, desc_hi, idesc, 1u);
                    tc_mma_lo_pair(acc, w1 + 6, t1 + 6, desc_hi, idesc, 1u);
                    tc_commit_pair_addr(empty_addr + slot8);
                } else {
                    tc_mma_lo(acc, w0, t0, desc_hi, idesc, first ? 0u : 1u);
                    tc_mma_lo(acc, w0 + 2, t0 + 2, desc_hi, idesc, 1u);
                    tc_mma_lo(acc, w0 + 4, t0 + 4, desc_hi, idesc, 1u);
                    tc_mma_lo(acc, w0 + 6, t0 + 6, desc_hi, idesc, 1u);
                    tc_mma_lo(acc, w1, t1, desc_hi, idesc, 1u);
                    tc_mma_lo(acc, w1 + 2, t1 + 2, desc_hi, idesc, 1u);
                    tc_mma_lo(acc, w1 + 4, t1 + 4, desc_hi, idesc, 1u);
                    tc_mma_lo(acc, w1 + 6, t1 + 6, desc_hi, idesc, 1u);
                    tc_commit_addr(empty_addr + slot8);
                }
                return true;
            };
            static_assert(NSLOT == 8 && BK == 64 && PRODUCERS == 2 && GROUP == 2, "the slot arithmetic and the MMAs of a group are written out");
            TileInfo next = tile_info<MAX_TOK, FEATS, PAIR>(p, unit, feat_tiles, rank);
            for (int tile = unit; tile < total_tiles && !*abort_flag; tile += n_units, local++) {
                const TileInfo t = next;
                if (tile + n_units < total_tiles) next = tile_info<MAX_TOK, FEATS, PAIR>(p, tile + n_units, feat_tiles, rank);
                const unsigned idesc = instr_desc(t.n_tok, PAIR ? 2 * BF : BF);
                const int buf = local % NBUF;
                // the epilogue must have emptied this accumulator buffer (NBUF tiles ago)
                if (!mbar_wait(&acc_empty_bar[buf], ((local / NBUF) & 1) ^ 1)) {
                    ok = false;
                    break;
                }
                tc_fence_after();
                const unsigned acc = tmem_base + buf * ACC_COLS;
                const int size_kb = (W_BYTES + (PAIR ? t.n_tok >> 1 : t.n_tok) * BK * 2) >> 10;
                int k = 0;
                if (step & 1) {                                       // the second k step of a group that the tile before began
                    ok = k_step(std::integral_constant<int, 1>{}, off1, acc, idesc, size_kb, true);
                    k = 1;
                }
                for (; k + 2 <= k_iters && ok; k += 2) ok = two_steps(acc, idesc, size_kb, k == 0);
                if (k < k_iters && ok)                                // the first k step of a group that the next tile ends, if there is one
                    ok = k_step(std::integral_constant<int, 0>{}, off0, acc, idesc, size_kb, k == 0);
                if (!ok || *abort_flag) break;
                if (PAIR) tc_commit_pair_addr(smem_u32(&acc_full_bar[buf]));
                else tc_commit(&acc_full_bar[buf]);                   // the accumulator is complete once all MMAs are done
            }
            if (!ok) {
                atomicOr(p.status, ESP_STATUS_WAIT_EXPIRED);
                *abort_flag = 1;
            }
        }
    } else {
        // Eight epilogue warps, two for each quarter of the TMEM lanes (a warp may read lanes 32*(warp%4)..+31
        // only): warps 2..5 take the even runs of 32 tokens, warps 7..10 the odd ones.  A store to global
        // memory keeps a warp for tens of cycles here, so the warps are what hides it.
        const int quad = warp & 3;
        const int half = warp >= 7 ? 1 : 0;
        int local = 0;
        TileInfo next = tile_info<MAX_TOK, FEATS, PAIR>(p, unit, feat_tiles, rank);
        for (int tile = unit; tile < total_tiles; tile += n_units, local++) {
            const TileInfo t = next;
            if (tile + n_units < total_tiles) next = tile_info<MAX_TOK, FEATS, PAIR>(p, tile + n_units, feat_tiles, rank);
            const int buf = local % NBUF;
            bool ok = !*abort_flag && mbar_wait(&acc_full_bar[buf], (local / NBUF) & 1);
            if (SWIGLU) {
                // the two warps of a pair meet at a named barrier for every run of tokens: they go on or leave together
                unsigned both;
                asm volatile(
                    "{\n.reg .pred p, q;\n"
                    "setp.ne.u32 p, %1, 0;\n"
                    "bar.red.and.pred q, %2, 64, p;\n"
                    "selp.u32 %0, 1, 0, q;\n}\n"
                    : "=r"(both) : "r"(ok ? 1u : 0u), "r"(1 + half * 2 + (quad & 1)) : "memory");
                ok = both != 0;
            }
            if (!ok) {
                if (lane == 0) {
                    atomicOr(p.status, ESP_STATUS_WAIT_EXPIRED);
                    *abort_flag = 1;
                }
                break;
            }
            tc_fence_after();
            const unsigned lane_addr = tmem_base + buf * ACC_COLS + ((unsigned)(quad * 32) << 16);
            if (SWIGLU) {
                // Lanes 0..63 hold the gate of 64 features, lanes 64..127 the up of the same features: the warp of
                // quad q (gate) and that of quad q + 2 (up) hold the two halves of every product.  Of each run of 32
                // tokens the gate warp finishes the first 16 and the up warp the last 16; each hands the other the
                // half it needs through shared memory (two buffers in turn, one named barrier per run).
                const int pair = quad & 1;
                const bool is_up = quad >= 2;
                const int f = t.f0 + pair * 32 + lane;
                const bool f_ok = f < p.N;
                bf16* out = reinterpret_cast<bf16*>(p.C);
                int flip = 0;
                for (int c0 = half * 32; c0 < t.n_tok; c0 += 64, flip ^= 1) {
                    float acc[32];
                    tc_ld32(lane_addr + c0, acc);
                    float* mine = swap + ((((half * 2 + flip) * 2 + pair) * 2 + (is_up ? 1 : 0)) * 16) * 32;
                    const float* theirs = swap + ((((half * 2 + flip) * 2 + pair) * 2 + (is_up ? 0 : 1)) * 16) * 32;
                    const int keep = is_up ? 16 : 0;                            // the up warp gives tokens 0..15 away
#pragma unroll
                    for (int i = 0; i < 16; i++) mine[i * 32 + lane] = is_up ? acc[i] : acc[16 + i];
                    asm volatile("bar.sync %0, 64;\n" ::"r"(1 + half * 2 + pair) : "memory");
#pragma unroll
                    for (int i = 0; i < 16; i++) {
                        const float other = theirs[i * 32 + lane];
                        const float own = is_up ? acc[16 + i] : acc[i];
                        const float g = is_up ? other : own, u = is_up ? own : other;
                        const int row = c0 + keep + i;
                        if (f_ok && row < t.n_rows)
                            out[(size_t)(t.row0 + row) * p.ldc + f] = __float2bfloat16_rn(__fdividef(g, 1.0f + __expf(-g)) * u);
                    }
                }
            } else {
                const int f = t.f0 + quad * 32 + lane;                    // this thread's output feature
                const bool f_ok = f < p.N;
                float* out = reinterpret_cast<float*>(p.C);
                for (int c0 = half * 32; c0 < t.n_tok; c0 += 64) {
                    float acc[32];
                    tc_ld32(lane_addr + c0, acc);
#pragma unroll
                    for (int i = 0; i < 32; i++) {
                        if (f_ok && c0 + i < t.n_rows) {
                            const float scale = p.row_scale ? p.row_scale[t.row0 + c0 + i] : 1.0f;
                            out[(size_t)(t.row0 + c0 + i) * p.ldc + f] = acc[i] * scale;
                        }
                    }
                }
            }
            // this warp has read its part of the buffer: hand it back to the MMA warp
            tc_fence_before();
            __syncwarp();
            if (lane == 0) {
                if (PAIR) mbar_arrive_leader(&acc_empty_bar[buf]);       // the leader's MMA thread waits for both CTAs' readers
                else mbar_arrive(&acc_empty_bar[buf]);
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (PAIR) cluster_sync_all();           // neither CTA gives up its shared or tensor memory while the other may still reach it
    if (warp == 1) {
        tc_fence_after();
        if (PAIR) asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"(TMEM_COLS));
        else asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"(TMEM_COLS));
    }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) != cudaSuccess ||
            qres != cudaDriverEntryPointSuccess)
            return nullptr;
        fn = reinterpret_cast<EncodeTiledFn>(ptr);
    }
    return fn;
}

// bfloat16 tensor [d2][d1][d0] (d0 innermost), box [1][box1][64], 128-byte swizzle, zero fill out of bounds
int make_map(CUtensorMap* map, const void* base, unsigned long long d0, unsigned long long d1, unsigned long long d2,
             unsigned box1, int rank) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return (int)cudaErrorNotSupported;
    const cuuint64_t dims[3] = {d0, d1, d2};
    const cuuint64_t strides[2] = {d0 * 2, d0 * d1 * 2};
    const cuuint32_t box[3] = {BK, box1, 1};
    const cuuint32_t elem[3] = {1, 1, 1};
    const CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, rank, const_cast<void*>(base), dims, strides, box, elem,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : (int)cudaErrorInvalidValue;
}
}  // namespace

// A [rows_total, K] bfloat16 (row-major, contiguous), W [G, w_rows, K] bfloat16.  Dense: tile_group = null,
// M rows.  Grouped: the token-tile list on the device (tiles of at most ``tile_max`` rows); ``max_tiles`` bounds
// their number.  swiglu: N is the intermediate size and w_rows = 2N.  K must be a multiple of 8, the
// bases 16-byte aligned.  pair: clusters of two CTAs share a token tile (tcgen05 cta_group::2): one MMA covers
// 256 weight rows, each CTA loads its own 128 and half of the token rows.
ESP_API int esp_gemm_tc05(const void* A, long long rows_total, const void* W, int groups, int w_rows,
                          const float* row_scale, void* C, long long ldc, const int* tile_group, const int* tile_row0,
                          const int* tile_rows, const int* n_tiles, int max_tiles, int tile_max, int M, int N, int K, int swiglu,
                          int pair, int max_ctas, int* status, cudaStream_t stream) {
    if (N <= 0 || K <= 0 || rows_total <= 0) return 0;
    if (max_ctas < 0 || (pair && max_ctas == 1)) return (int)cudaErrorInvalidValue;
    if (K % 8 != 0 || ((uintptr_t)A & 15) || ((uintptr_t)W & 15)) return (int)cudaErrorInvalidValue;
    CUtensorMap map_a, map_a64, map_a128, map_w;
    int rc = make_map(&map_a, A, (unsigned long long)K, (unsigned long long)rows_total, 1, TOK_BOX, 3);
    if (rc) return rc;
    rc = make_map(&map_a64, A, (unsigned long long)K, (unsigned long long)rows_total, 1, 64, 3);
    if (rc) return rc;
    rc = make_map(&map_a128, A, (unsigned long long)K, (unsigned long long)rows_total, 1, 128, 3);
    if (rc) return rc;
    // the weights always use a 3-D map so that the kernel has one code path; a dense product is one group
    rc = make_map(&map_w, W, (unsigned long long)K, (unsigned long long)w_rows, (unsigned long long)groups, swiglu ? BF / 2 : BF, 3);
    if (rc) return rc;
    Tc05Params p{tile_group, tile_row0, tile_rows, n_tiles, row_scale, C, ldc, M, N, K, status};
    // ``tile_max``: the most rows a tile of the list has, 128 or 256 (with 256 an expert's weights pass once
    // for up to 256 of its rows); dense products cut tiles of 256 rows (MMAs of N = 256 run at the full rate)
    if (tile_group && tile_max != 128 && tile_max != 256) return (int)cudaErrorInvalidValue;
    const int max_tok = tile_group ? tile_max : 256;
    const int token_tiles = tile_group ? max_tiles : (M + max_tok - 1) / max_tok;     // upper bound when grouped
    if (token_tiles <= 0) return 0;
    const int feats = swiglu ? BF / 2 : BF;
    const long long tiles_bound = (long long)token_tiles * ((N + feats - 1) / feats);
    static int sm_count = 0;
    if (!sm_count) {
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev);
        if (sm_count <= 0) sm_count = 148;
    }
    // ``max_ctas`` > 0: the kernel takes at most that many SMs (its CTAs walk the tiles with the grid's stride),
    // so that kernels of another stream find room beside it
    const int ctas = max_ctas > 0 && max_ctas < sm_count ? max_ctas : sm_count;
    const size_t smem = PRODUCERS * RING_BYTES + 1024 + BAR_BYTES + SWAP_BYTES;     // 230,656 of the 232,448 bytes a block may have
    const int which = (pair ? 4 : 0) + (swiglu ? 2 : 0) + (max_tok == 256 ? 1 : 0);
    typedef void (*Kernel)(const CUtensorMap, const CUtensorMap, const CUtensorMap, const CUtensorMap, Tc05Params);
    static const Kernel kernels[8] = {
        gemm_tc05_kernel<false, 128, false>, gemm_tc05_kernel<false, 256, false>, gemm_tc05_kernel<true, 128, false>,
        gemm_tc05_kernel<true, 256, false>,  gemm_tc05_kernel<false, 128, true>,  gemm_tc05_kernel<false, 256, true>,
        gemm_tc05_kernel<true, 128, true>,   gemm_tc05_kernel<true, 256, true>};
    static bool raised[8] = {false, false, false, false, false, false, false, false};
    if (!raised[which]) {
        cudaError_t e = cudaFuncSetAttribute(kernels[which], cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        raised[which] = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.blockDim = dim3(THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    if (pair) {
        // two CTAs of a cluster share a token tile: the grid is a whole number of pairs, one pair per two SMs
        const long long pair_tiles = (long long)token_tiles * (((N + feats - 1) / feats + 1) / 2);
        const long long pairs = pair_tiles < ctas / 2 ? pair_tiles : ctas / 2;
        cfg.gridDim = dim3((unsigned)(2 * pairs));
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = 2;
        attr[0].val.clusterDim.y = 1;
        attr[0].val.clusterDim.z = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
    } else {
        cfg.gridDim = dim3((unsigned)(tiles_bound < ctas ? tiles_bound : ctas));
    }
    cudaLaunchKernelEx(&cfg, kernels[which], map_a, map_a64, map_a128, map_w, p);
    return esp_launch_status();
}

// ---------------------------------------------------------------------------------------------------
// A probe of the bounded wait that every kernel of this library relies on: one thread waits, for at most
// ``polls`` tries, on an mbarrier that nothing will ever complete (no copy is in flight, nobody arrives),
// then reports ESP_STATUS_WAIT_EXPIRED and returns.  It shows that a wait that runs out ends the kernel in an
// orderly way and leaves the device usable.  ``polls`` is clamped to 2^20.
__global__ void wait_probe_kernel(unsigned polls, int* __restrict__ status) {
    __shared__ __align__(8) unsigned long long bar;
    if (threadIdx.x == 0) {
        tc05::mbar_init(&bar, 1);
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
        if (!tc05::mbar_wait_limited(&bar, 0, polls)) atomicOr(status, ESP_STATUS_WAIT_EXPIRED);
    }
}

ESP_API int esp_wait_probe(int polls, int* status, cudaStream_t stream) {
    if (polls <= 0) return (int)cudaErrorInvalidValue;
    wait_probe_kernel<<<1, 32, 0, stream>>>((unsigned)(polls > (1 << 20) ? (1 << 20) : polls), status);
    return esp_launch_status();
}
