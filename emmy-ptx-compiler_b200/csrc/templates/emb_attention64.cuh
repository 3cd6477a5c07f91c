// FlashAttention-2-style forward template for sm_100a on 64-KEY tiles with the scores DOUBLE-BUFFERED in tensor
// memory. Same work items, online update and masking rules as emb_attention.cuh (which walks 128-key tiles and
// keeps one score buffer per query tile); what changes is the dependency chain of one query tile:
//
//   emb_attention.cuh    S(j) -> softmax(j) -> P(j) over S's columns -> PV(j) -> QK(j+1) -> S(j+1) -> softmax(j+1) ...
//                        the softmax warps of a query tile idle during PV(j) and QK(j+1): P(j) lives in S's own columns,
//                        so the next scores cannot be written before PV(j) has read it.
//   here                 two score buffers of 64 columns per query tile. QK(j+2) is issued right after PV(j) into the
//                        buffer PV(j) has just read, so S(j+1) is complete BEFORE softmax(j) ends and the softmax
//                        warps go from one tile to the next without waiting for the tensor pipe.
//
// Warps: 0 scheduler + TMA producer; 1 .. NQ one MMA issuer PER query tile; then one softmax warp group (SPLIT = 1) or two
// (SPLIT = 2) per query tile. A lone issuer for both query tiles was the bottleneck of the first version of this file: a
// thread needs about 35 cycles per tcgen05.mma it issues, a 128 x 64 x 16 product occupies the tensor pipe for 32 to 48, and
// time stamps taken in the kernel (clock register, one CTA, 32 key tiles) showed the softmax warps waiting 600 cycles per
// tile for scores whose instructions had not been issued yet.
//
// What bounds it now, from the same kind of time stamps: a softmax warp's 64-key step takes about 1700 cycles, of which the
// exponentials take 1000 to 1250 (the two query tiles' warps of one 32-row quarter share a scheduler and its SFU, 4 results
// per clock: 2 x 64 x 32 / 4 = 1024 cycles), the maximum 200, and reading, storing and the barriers 300; the schedulers that
// also host an issuer warp are the slowest (1250 against 1016), and every tile waits for its slowest quarter. Without the
// weights' loop the kernel takes 834 us on the causal 8 x 32 x 4096 x 128 workload (the tensor pipe's share: Q K^T with
// N = 64 reads 6 KB of shared memory per 32 cycles of arithmetic), with it about 1000 us.
//
// Tensor memory (512 columns): S(i, b) at (2 i + b) * 64 for query tile i, buffer b; O_i at 256 + 128 i. A tile's 64
// scores of a row fit two register chunks, so the maximum and the weights come from ONE read of tensor memory.
// K and V tiles are 64 keys x D (8 KB per 64-wide d half), four stages each.
//
// SPLIT = 2 puts TWO softmax warp groups on a query tile: the two threads of a row take 32 scores each, exchange their
// maxima (and, at the end of an item, their sums) through shared memory behind a two-arrival mbarrier per 32-row
// quarter, and each rescales and stores half of the row's output columns. Measured slower than SPLIT = 1 (1090 against
// 998 us): the schedulers were not short of warps, and the exchange adds to every step.
#pragma once
#include "emb_attention.cuh"

namespace emb {

template <int NQ, bool CAUSAL, bool BF16, int POLY_PERIOD, bool MASKED = false, int D = 128, int SPLIT = 1>
__device__ __forceinline__ void attention_fwd_kernel64(const CUtensorMap* __restrict__ map_q, const CUtensorMap* __restrict__ map_k,
                                                       const CUtensorMap* __restrict__ map_v, void* __restrict__ o_out,
                                                       AttnShape shape, unsigned* status, const float* __restrict__ mask = nullptr) {
    constexpr int BM = 128, BN = 64, UMMA_K = 16, HALVES = D / 64;
    static_assert(D == 64 || D == 128, "head dimension 64 or 128");
    static_assert(NQ == 1 || NQ == 2, "one or two query tiles per CTA");
    static_assert(SPLIT == 1 || SPLIT == 2, "one or two threads per query row");
    constexpr int COLS = BN / SPLIT;                     // scores of a key tile per thread
    constexpr int OC = D / SPLIT;                        // output columns per thread
    constexpr uint32_t Q_HALF = 128 * 64 * 2;            // a 128-row x 64-column 16-bit box: 16 KB
    constexpr uint32_t Q_TILE = HALVES * Q_HALF;
    constexpr uint32_t KV_HALF = 64 * 64 * 2;            // a 64-key x 64-column box: 8 KB
    constexpr uint32_t KV_TILE = HALVES * KV_HALF;
    constexpr int KS = 4;                                // stages of K and of V
    constexpr uint32_t TMEM_COLS = 512, O_COL = 256;
    using out_t = typename Half16<BF16>::type;

    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* q_smem = smem;
    uint8_t* k_smem = q_smem + NQ * Q_TILE;
    uint8_t* v_smem = k_smem + KS * KV_TILE;
    uint64_t* bars = reinterpret_cast<uint64_t*>(v_smem + KS * KV_TILE);
    uint64_t* q_full = bars;                  // 1
    uint64_t* q_empty = bars + 1;             // 1: the item's last Q K^T has read the Q tiles
    uint64_t* k_full = bars + 2;              // KS
    uint64_t* k_empty = k_full + KS;
    uint64_t* v_full = k_empty + KS;
    uint64_t* v_empty = v_full + KS;
    uint64_t* s_full = v_empty + KS;          // 4: query tile i, buffer b at [2 i + b]
    uint64_t* p_ready = s_full + 4;           // 4: the weights of the tile in buffer [2 i + b] are in tensor memory (4 warps)
    uint64_t* o_done = p_ready + 4;           // 2: P V of a key tile has completed
    uint64_t* o_final = o_done + 2;           // 2: P V of an item's LAST key tile has completed
    uint64_t* item_full = o_final + 2;        // 2
    uint64_t* item_empty = item_full + 2;     // 2
    uint64_t* x_bar = item_empty + 2;         // 8: the two warps of (query tile i, quarter q) at [4 i + q] have written their halves
    uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(x_bar + 8);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);
    volatile int* item_ring = abort_flag + 1;
    float* x_buf = reinterpret_cast<float*>(bars + 64);  // [query tile][slot][half][row]: what the halves of a row tell each other
    const tc::Guard guard{status, abort_flag};

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int q_blocks = (shape.seq + NQ * BM - 1) / (NQ * BM);
    const int kv_tiles = (shape.seq + BN - 1) / BN;
    const int num_items = shape.batch_heads * q_blocks;
    unsigned* work_counter = status + 4;  // zero at launch; the last CTA to finish resets it (and status[5])

    struct Item {
        int q0, bh, row_base, n_kv[NQ], n_max;
    };
    auto decode = [&](int w) {
        Item it;
        // work-item order: the blocks of one head together, longest first (its K and V stay in L2 while its blocks run), or,
        // when every head's K and V fit L2 at once, the longest blocks of ALL heads first (a better balanced end of the launch)
        const int bh = shape.longest_first ? w % shape.batch_heads : w / q_blocks;
        const int qb = q_blocks - 1 - (shape.longest_first ? w / shape.batch_heads : w % q_blocks);
        it.q0 = qb * NQ * BM;
        it.bh = bh;
        it.row_base = bh * shape.seq;
#pragma unroll
        for (int i = 0; i < NQ; ++i) it.n_kv[i] = CAUSAL ? min(kv_tiles, (it.q0 + i * BM + BM) / BN) : kv_tiles;
        it.n_max = it.n_kv[NQ - 1];
        return it;
    };

    if (threadIdx.x == 0) {
        tc::mbar_init(q_full, 1);
        tc::mbar_init(q_empty, NQ);  // every issuer
        for (int s = 0; s < KS; ++s) {
            tc::mbar_init(&k_full[s], 1);
            tc::mbar_init(&k_empty[s], NQ);
            tc::mbar_init(&v_full[s], 1);
            tc::mbar_init(&v_empty[s], NQ);
        }
        // A waiter on a phase's parity must never be two phases behind the barrier. The softmax warps run up to two key
        // tiles ahead of the MMA thread (both score buffers), so what they signal per tile (p_ready) and what they wait for
        // per tile (s_full) are barriers PER BUFFER, each completing every second tile; o_done, one phase per tile, is
        // only waited for one tile back (the rescale), and an item's last product has a barrier of its own (o_final).
        for (int i = 0; i < 4; ++i) {
            tc::mbar_init(&s_full[i], 1);
            tc::mbar_init(&p_ready[i], 4 * SPLIT);
        }
        for (int i = 0; i < 8; ++i) tc::mbar_init(&x_bar[i], 2);
        for (int i = 0; i < 2; ++i) {
            tc::mbar_init(&o_done[i], 1);
            tc::mbar_init(&o_final[i], 1);
            tc::mbar_init(&item_full[i], 1);
            tc::mbar_init(&item_empty[i], NQ + 4 * SPLIT * NQ);  // every issuer and every softmax warp
        }
        *abort_flag = 0;
        tc::mbar_init_fence();
        tc::tma_prefetch_desc(map_q);
        tc::tma_prefetch_desc(map_k);
        tc::tma_prefetch_desc(map_v);
    }
    if (warp == 1) tc::tmem_alloc(tmem_holder, TMEM_COLS);
    tc::tc_fence_before_sync();
    __syncthreads();
    tc::tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_holder;

    if (warp == 0) {
        // ---------------------------------------------------------------- scheduler + producer
        if (lane == 0) {
            uint32_t kvc = 0;  // K/V tiles loaded so far, over all items
            for (uint32_t it = 0;; ++it) {
                const uint32_t slot = it & 1;
                if (!tc::mbar_wait(&item_empty[slot], ((it >> 1) & 1) ^ 1, guard, tc::WAIT_OTHER, it)) break;
                const unsigned claimed = atomicAdd(work_counter, 1u);
                const int w = claimed < static_cast<unsigned>(num_items) ? static_cast<int>(claimed) : -1;
                item_ring[slot] = w;
                tc::mbar_arrive(&item_full[slot]);
                if (w < 0) break;
                const Item item = decode(w);
                bool alive = true;
                for (int j = 0; alive && j < item.n_max; ++j, ++kvc) {
                    const uint32_t s = kvc % KS, ph = (kvc / KS) & 1;
                    if (!tc::mbar_wait(&k_empty[s], ph ^ 1, guard, tc::WAIT_SMEM_EMPTY, j)) { alive = false; break; }
                    tc::mbar_arrive_expect_tx(&k_full[s], KV_TILE);
#pragma unroll
                    for (int h = 0; h < HALVES; ++h)
                        tc::tma_load_3d(k_smem + s * KV_TILE + h * KV_HALF, map_k, &k_full[s], h * 64, j * BN, item.bh);
                    if (j == 0) {  // Q right behind the first K: the first scores need both
                        if (!tc::mbar_wait(q_empty, (it & 1) ^ 1, guard, tc::WAIT_SMEM_EMPTY, 9000)) { alive = false; break; }
                        tc::mbar_arrive_expect_tx(q_full, NQ * Q_TILE);
#pragma unroll
                        for (int i = 0; i < NQ; ++i)
#pragma unroll
                            for (int h = 0; h < HALVES; ++h)
                                tc::tma_load_3d(q_smem + i * Q_TILE + h * Q_HALF, map_q, q_full, h * 64, item.q0 + i * BM, item.bh);
                    }
                    if (!tc::mbar_wait(&v_empty[s], ph ^ 1, guard, tc::WAIT_SMEM_EMPTY, 1000 + j)) { alive = false; break; }
                    tc::mbar_arrive_expect_tx(&v_full[s], KV_TILE);
#pragma unroll
                    for (int h = 0; h < HALVES; ++h)
                        tc::tma_load_3d(v_smem + s * KV_TILE + h * KV_HALF, map_v, &v_full[s], h * 64, j * BN, item.bh);
                }
                if (!alive) break;
            }
        }
    } else if (warp <= NQ) {
        // ---------------------------------------------------------------- MMA issuers: warp 1 + i for query tile i
        // One issuer per query tile: a thread needs some 35 cycles per tcgen05.mma of 128 x 64 x 16 (32 cycles of tensor
        // pipe), so ONE thread issuing both tiles' products kept the pipe waiting for instructions. The two issuers share
        // the K and V stages and the Q tiles, whose "empty" barriers count one arrival per issuer.
        if (tc::elect_one()) {
            const int i = warp - 1;
            constexpr uint32_t idesc_qk = tc::idesc_f16(BM, BN, BF16);
            constexpr uint32_t idesc_pv = tc::idesc_f16(BM, D, BF16) | (1u << 16);  // B (= V) is MN-major
            const uint64_t qd = tc::smem_desc_k128(q_smem + i * Q_TILE);
            const uint32_t s_col = tmem_base + 2 * i * BN, o_col = tmem_base + O_COL + i * 128;
            uint32_t kvc = 0;  // K/V tiles of the items before this one
            uint32_t c = 0;    // Q K^T issued, over all items: buffer and phase of s_full
            uint32_t pv = 0;   // P V issued, over all items: buffer and phase of p_ready
            bool alive = true;
            for (uint32_t it = 0; alive; ++it) {
                const uint32_t slot = it & 1;
                if (!tc::mbar_wait(&item_full[slot], (it >> 1) & 1, guard, tc::WAIT_OTHER, 100 + it)) break;
                const int w = item_ring[slot];
                tc::mbar_arrive(&item_empty[slot]);
                if (w < 0) break;
                const Item item = decode(w);
                const int n_mine = item.n_kv[i];
                if (!tc::mbar_wait(q_full, it & 1, guard, tc::WAIT_SMEM_FULL, 9999)) break;

                // S(buffer) = Q_i K_j^T over d in 16-wide steps
                auto issue_qk = [&](int j) {
                    const uint32_t t = kvc + j, s = t % KS;
                    if (!tc::mbar_wait(&k_full[s], (t / KS) & 1, guard, tc::WAIT_SMEM_FULL, j)) return false;
                    tc::tc_fence_after_sync();
                    const uint32_t b = c & 1;
                    // (a descriptor's low bits are the address in 16-byte units: steps inside a tile are plain additions)
                    const uint64_t kd = tc::smem_desc_k128(k_smem + s * KV_TILE);
#pragma unroll
                    for (int kk = 0; kk < D / UMMA_K; ++kk)
                        tc::mma_f16_ss(s_col + b * BN, qd + (((kk / 4) * Q_HALF + (kk % 4) * (UMMA_K * 2)) >> 4),
                                       kd + (((kk / 4) * KV_HALF + (kk % 4) * (UMMA_K * 2)) >> 4), idesc_qk, kk != 0);
                    tc::mma_commit(&s_full[2 * i + b]);
                    ++c;
                    tc::mma_commit(&k_empty[s]);
                    if (j == n_mine - 1) tc::mma_commit(q_empty);  // this tile's last use of Q in the item
                    return true;
                };
                // O_i += P_i V_j: P from the buffer's first 32 columns, V_j [key][d] MN-major (64-wide d halves KV_HALF apart)
                auto issue_pv = [&](int j) {
                    const uint32_t t = kvc + j, s = t % KS;
                    if (!tc::mbar_wait(&v_full[s], (t / KS) & 1, guard, tc::WAIT_SMEM_FULL, 1000 + j)) return false;
                    tc::tc_fence_after_sync();
                    const uint32_t b = pv & 1;
                    const uint64_t vd = tc::smem_desc_mn128(v_smem + s * KV_TILE, KV_HALF);
#pragma unroll
                    for (int kk = 0; kk < BN / UMMA_K; ++kk)
                        tc::mma_f16_ts(o_col, s_col + b * BN + kk * (UMMA_K / 2), vd + ((kk * UMMA_K * 128) >> 4), idesc_pv, (j | kk) != 0);
                    tc::mma_commit(&o_done[i]);
                    if (j == n_mine - 1) tc::mma_commit(&o_final[i]);
                    ++pv;
                    tc::mma_commit(&v_empty[s]);
                    return true;
                };
                // a key tile this query tile does not read (past its diagonal) is still released by this issuer, and only
                // once it is loaded: an arrival ahead of the load could complete the stage's PREVIOUS phase, which the other
                // issuer may still be reading
                auto skip = [&](int j) {
                    const uint32_t t = kvc + j, s = t % KS;
                    if (!tc::mbar_wait(&k_full[s], (t / KS) & 1, guard, tc::WAIT_SMEM_FULL, 7000 + j)) return false;
                    tc::mbar_arrive(&k_empty[s]);
                    if (!tc::mbar_wait(&v_full[s], (t / KS) & 1, guard, tc::WAIT_SMEM_FULL, 8000 + j)) return false;
                    tc::mbar_arrive(&v_empty[s]);
                    return true;
                };

                // two score tiles ahead
                for (int j = 0; alive && j < 2 && j < n_mine; ++j) alive = issue_qk(j);
                for (int j = 0; alive && j < n_mine; ++j) {
                    if (!tc::mbar_wait(&p_ready[2 * i + (pv & 1)], (pv >> 1) & 1, guard, tc::WAIT_TMEM_FULL, 2500 + j)) { alive = false; break; }
                    alive = issue_pv(j);
                    // the buffer P V (j) has just read is the one S(j + 2) goes to: the tensor pipe runs one thread's products in order
                    if (alive && j + 2 < n_mine) alive = issue_qk(j + 2);
                }
                for (int j = n_mine; alive && j < item.n_max; ++j) alive = skip(j);
                kvc += item.n_max;
            }
        }
    } else {
        // ---------------------------------------------------------------- softmax, correction, epilogue
        const int i = (warp - 1 - NQ) / (4 * SPLIT);       // query tile of this warp
        const int half = SPLIT == 2 ? ((warp - 1 - NQ) >> 2) & 1 : 0;  // which scores of a row and which output columns are this thread's
        const int quarter = warp & 3;        // the TMEM lanes this warp may touch: 32 * quarter ..
        const int row = quarter * 32 + lane; // row of the query tile
        const uint32_t lane_addr = static_cast<uint32_t>(quarter * 32) << 16;
        const uint32_t o_addr = tmem_base + lane_addr + O_COL + i * 128 + half * OC;
        uint32_t steps = 0;  // key tiles this query tile has processed, over all items
        uint32_t xc = 0;     // exchanges with the row's other thread so far: slot and phase of x_bar
        bool alive = i < NQ;
        // the row's other thread gets `mine` and this one gets the other's: both write, both arrive, both wait, both read.
        // The slot alternates, so a thread that runs on to its next exchange writes where its partner has already read.
        auto exchange = [&](float mine, float& other, unsigned detail) {
            float* slot = x_buf + ((i * 2 + (xc & 1)) * 2) * BM;
            slot[half * BM + row] = mine;
            __syncwarp();
            if (lane == 0) tc::mbar_arrive(&x_bar[4 * i + quarter]);
            if (!tc::mbar_wait(&x_bar[4 * i + quarter], xc & 1, guard, tc::WAIT_OTHER, detail)) return false;
            other = slot[(half ^ 1) * BM + row];
            ++xc;
            return true;
        };
        for (uint32_t it = 0; alive; ++it) {
            const uint32_t slot = it & 1;
            if (!tc::mbar_wait(&item_full[slot], (it >> 1) & 1, guard, tc::WAIT_OTHER, 200 + it)) break;
            const int w = item_ring[slot];
            __syncwarp();
            if (lane == 0) tc::mbar_arrive(&item_empty[slot]);
            if (w < 0) break;
            const Item item = decode(w);
            const int n_mine = item.n_kv[i < NQ ? i : 0];
            const int q_row = item.q0 + i * BM + row;
            const int row_base = item.row_base;
            // the reference maximum, in units of log2, seeded like the interpreter's maximum fold (-1e30, finite): a first key
            // tile whose scores are all -inf (an additive mask) then gives weights 2^(-inf + 1e30) = 0, not NaN
            float m_used = -1e30f;
            float l = 0.0f;
            for (int j = 0; alive && j < n_mine; ++j, ++steps) {
                const uint32_t b = steps & 1;
                const uint32_t s_addr = tmem_base + lane_addr + (2 * i + b) * BN;
                if (!tc::mbar_wait(&s_full[2 * i + b], (steps >> 1) & 1, guard, tc::WAIT_TMEM_FULL, 3000 + j)) {
                    alive = false;
                    break;
                }
                tc::tc_fence_after_sync();
                uint32_t sr[COLS / 32][32];  // this thread's scores of the tile: read once
#pragma unroll
                for (int c = 0; c < COLS / 32; ++c) tc::tmem_ld_32x32(s_addr + half * COLS + c * 32, sr[c]);
                // keys beyond the query (causal) or beyond the end of the head score -inf: only columns <= limit are visible
                const int first = j * BN + half * COLS;  // key of this thread's first score
                const int past_end = shape.seq - 1 - first;
                const int limit = CAUSAL ? min(q_row - first, past_end) : past_end;
                const bool masked_tile = limit < COLS - 1;
                tc::tmem_ld_wait();
#pragma unroll
                for (int c = 0; c < COLS / 32; ++c) {
                    if (MASKED) {
#pragma unroll
                        for (int x = 0; x < 32; ++x) {
                            const int key = min(first + c * 32 + x, shape.seq - 1);
                            sr[c][x] = __float_as_uint(fmaf(__ldg(mask + key), shape.inv_scale, __uint_as_float(sr[c][x])));
                        }
                    }
                    if (masked_tile) {
#pragma unroll
                        for (int x = 0; x < 32; ++x)
                            if (c * 32 + x > limit) sr[c][x] = 0xff800000u;
                    }
                }
                // the row maximum (independent chains)
                float mx8[8];
#pragma unroll
                for (int u = 0; u < 8; ++u) mx8[u] = -__int_as_float(0x7f800000);
#pragma unroll
                for (int c = 0; c < COLS / 32; ++c)
#pragma unroll
                    for (int x = 0; x < 32; x += 4)
                        mx8[(x / 4) & 7] = emb::max3(mx8[(x / 4) & 7], emb::max3(__uint_as_float(sr[c][x]), __uint_as_float(sr[c][x + 1]),
                                                                                 __uint_as_float(sr[c][x + 2])),
                                                     __uint_as_float(sr[c][x + 3]));
                float mx = fmaxf(emb::max3(mx8[0], mx8[1], mx8[2]), emb::max3(emb::max3(mx8[3], mx8[4], mx8[5]), mx8[6], mx8[7]));
                if (SPLIT == 2) {
                    // (the partner's weights go over score columns this thread has just read: the exchange orders the two)
                    float theirs;
                    if (!exchange(mx, theirs, 6000 + j)) {
                        alive = false;
                        break;
                    }
                    mx = fmaxf(mx, theirs);
                }
                const float m_new = fmaxf(m_used, mx * shape.scale_log2);
                // move the reference maximum only when it grew by more than 8 (a factor 256)
                const bool moved = m_new - m_used > 8.0f;
                if (__any_sync(0xffffffffu, moved) && j > 0) {
                    const float alpha = moved ? emb::ex2_approx_ftz(m_used - m_new) : 1.0f;
                    // O must hold P V (i, j - 1) before it is rescaled: unlike the scores, that product may still be running
                    if (!tc::mbar_wait(&o_done[i], (steps - 1) & 1, guard, tc::WAIT_TMEM_EMPTY, 4000 + j)) {
                        alive = false;
                        break;
                    }
                    tc::tc_fence_after_sync();
#pragma unroll 1
                    for (int c = 0; c < OC / 32; ++c) {
                        uint32_t orow[32];
                        tc::tmem_ld_32x32(o_addr + c * 32, orow);
                        tc::tmem_ld_wait();
#pragma unroll
                        for (int x = 0; x < 32; ++x) orow[x] = __float_as_uint(__uint_as_float(orow[x]) * alpha);
                        tc::tmem_st_32x32(o_addr + c * 32, orow);
                    }
                    tc::tmem_st_wait();
                    l *= alpha;
                }
                if (moved) m_used = m_new;
                // weights 2^(s * scale - m), their sum, and P as 16-bit pairs over the buffer's first 32 columns
                const unsigned long long neg_m2 = emb::pack_f2(-m_used, -m_used);
                const unsigned long long scale2 = emb::pack_f2(shape.scale_log2, shape.scale_log2);
                unsigned long long sum2[2] = {emb::pack_f2(0.0f, 0.0f), emb::pack_f2(0.0f, 0.0f)};
#pragma unroll
                for (int c = 0; c < COLS / 32; ++c) {
                    uint32_t packed[16];
#pragma unroll
                    for (int x = 0; x < 32; x += 2) {
                        const unsigned long long t2 =
                            emb::fma_f2(emb::pack_f2(__uint_as_float(sr[c][x]), __uint_as_float(sr[c][x + 1])), scale2, neg_m2);
                        float t0, t1, p0, p1;
                        emb::unpack_f2(t2, t0, t1);
                        if (POLY_PERIOD > 0 && ((c * 16 + x / 2) % (POLY_PERIOD > 0 ? POLY_PERIOD : 1)) == POLY_PERIOD - 1) {
                            emb::ex2_poly3_pair(t0, t1, p0, p1);  // this pair's exponentials on the FMA pipe, not the SFU
                        } else {
                            p0 = emb::ex2_approx_ftz(t0);
                            p1 = emb::ex2_approx_ftz(t1);
                        }
                        sum2[(x / 2) & 1] = emb::add_f2(sum2[(x / 2) & 1], emb::pack_f2(p0, p1));
                        packed[x / 2] = pack2<BF16>(p0, p1);
                    }
                    asm volatile(
                        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
                        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};" ::"r"(s_addr + (half * (COLS / 32) + c) * 16),
                        "r"(packed[0]), "r"(packed[1]), "r"(packed[2]), "r"(packed[3]), "r"(packed[4]), "r"(packed[5]),
                        "r"(packed[6]), "r"(packed[7]), "r"(packed[8]), "r"(packed[9]), "r"(packed[10]), "r"(packed[11]),
                        "r"(packed[12]), "r"(packed[13]), "r"(packed[14]), "r"(packed[15])
                        : "memory");
                }
                float sum, sum_hi;
                emb::unpack_f2(emb::add_f2(sum2[0], sum2[1]), sum, sum_hi);
                sum += sum_hi;
                l += sum;
                tc::tmem_st_wait();
                tc::tc_fence_before_sync();
                __syncwarp();
                if (lane == 0) tc::mbar_arrive(&p_ready[2 * i + b]);
            }
            if (SPLIT == 2 && alive) {  // the row's sum is the two halves'
                float theirs;
                if (exchange(l, theirs, 7000)) l += theirs; else alive = false;
            }
            // the item's last P V (its two last ones may still be running when the softmax of the last tile ends)
            if (alive && tc::mbar_wait(&o_final[i], it & 1, guard, tc::WAIT_TMEM_EMPTY, 5000)) {
                tc::tc_fence_after_sync();
                const float inv = 1.0f / l;
                out_t* dst = static_cast<out_t*>(o_out) + (static_cast<size_t>(row_base) + q_row) * D + half * OC;
#pragma unroll 1
                for (int c = 0; c < OC / 32; ++c) {
                    uint32_t orow[32];
                    tc::tmem_ld_32x32(o_addr + c * 32, orow);
                    tc::tmem_ld_wait();
                    if (q_row >= shape.seq) continue;  // a row past the end of the head (partial last query tile)
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        uint4 v;
                        v.x = pack2<BF16>(__uint_as_float(orow[8 * q + 0]) * inv, __uint_as_float(orow[8 * q + 1]) * inv);
                        v.y = pack2<BF16>(__uint_as_float(orow[8 * q + 2]) * inv, __uint_as_float(orow[8 * q + 3]) * inv);
                        v.z = pack2<BF16>(__uint_as_float(orow[8 * q + 4]) * inv, __uint_as_float(orow[8 * q + 5]) * inv);
                        v.w = pack2<BF16>(__uint_as_float(orow[8 * q + 6]) * inv, __uint_as_float(orow[8 * q + 7]) * inv);
                        *reinterpret_cast<uint4*>(dst + c * 32 + 8 * q) = v;
                    }
                }
            } else {
                alive = false;
            }
        }
    }

    tc::tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        tc::tc_fence_after_sync();
        tc::tmem_dealloc(tmem_base, TMEM_COLS);
    }
    if (threadIdx.x == 0) {
        // every CTA has drawn its end-of-work token before it gets here: the last one re-arms the counters for the next launch
        __threadfence();
        if (atomicAdd(status + 5, 1u) == gridDim.x - 1) {
            status[4] = 0;
            status[5] = 0;
            __threadfence();
        }
    }
}

}  // namespace emb
