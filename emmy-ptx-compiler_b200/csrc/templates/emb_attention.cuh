// FlashAttention-2-style forward template for sm_100a: O = softmax(scale * Q K^T [causal]) V for
// head dimension 128, 16-bit Q/K/V/O, f32 scores and accumulators in tensor memory.
//
// It takes the place of the reference's lane-blocked SIMT attention: there the online-softmax update
// found in the IR (emmy_ptx/mapping.py:402-500) is re-blocked over G <= 32 keys, the scores are
// computed once per key block on the lanes of a row and broadcast through shared memory
// (emmy_ptx/mapping.py:665-820, emmy_ptx/lanes.py:293-346, 610-658), all with scalar FMAs and one exp
// per key (emmy_ptx/mathlib.py:111-136). Here persistent CTAs (one per SM) claim work items from a counter in
// global memory; an item is NQ = 2 query tiles of 128 rows of one (batch, head), against which the CTA streams
// 128-key tiles of K and V. The roles run ahead of each other ACROSS items: the next item's loads and first
// score tiles are in flight while the softmax warps still normalise and store the previous item's output.
//
//   warp 0      one thread claims items (atomicAdd; heaviest first within a head, the heads in order so that the
//               CTAs running together share K and V in L2), publishes them to the other roles through a two-slot
//               ring, and issues the TMA tensor-map loads (128-byte swizzle, no multicast): Q per item, K_j and
//               V_j into two stages each, completion on mbarriers
//   warp 1      one thread issues tcgen05.mma: S_i = Q_i K_j^T (operands in shared memory) and
//               O_i += P_i V_j (P_i read from TENSOR memory, V_j MN-major from shared memory); both
//               query tiles alternate, so the tensor pipe works on one while the other is in softmax
//   warps 2-5   softmax of query tile 0: one thread per row reads its 128 scores from TMEM, keeps the
//   warps 6-9   running maximum and sum, writes P as 16-bit pairs over S's columns, rescales the O
//   (tile 1)    accumulator in TMEM only when the maximum moved by more than 2^8 (the final division by
//               the running sum makes the stale maximum exact), and at the end normalises and stores O
//
// The online update is the IR's (state m, l, o; alpha = exp(m - m'), beta = exp(s - m')); it is applied
// once per 128-key tile instead of once per key, and in base 2 (scale * log2 e folded into one FMA).
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "emb_gemm.cuh"
#include "emb_math.cuh"

namespace emb {

struct AttnShape {
    int batch_heads;   // batch * heads
    int seq;           // queries = keys per (batch, head); any count: a partial last tile's key slots score -inf
                       // (as the reference fills the slots past the end of its last key block, emmy_ptx/mapping.py:743-754)
    float scale_log2;  // softmax scale * log2(e)
    float inv_scale;   // 1 / softmax scale (used with a mask only)
    int longest_first; // work items ordered by length over all heads (else head by head)
};

// The tensor maps are three-dimensional, (d, row of the head, head): rows past the end of a head read as zeros,
// never as the next head's rows. MASKED: `mask` holds one f32 per key, added to every query's scaled score of
// that key before the softmax (emmy's additive mask, tests/test_gpu_lowering.py:256-306 of the reference).
// OPTIMISTIC: from an item's second key tile on, the tile's row maximum is not found by a pass of its own over the
// scores in tensor memory: the weights are taken against the reference maximum carried from the earlier tiles while the
// tile's own maximum is tracked, and the reference moves lazily before the NEXT tile (the final division by the
// running sum makes any reference exact as long as nothing overflows). A score that exceeds the reference by more
// than 2^15 - which would overflow a 16-bit weight - is caught chunk by chunk before its weight is made: the reference
// then moves at once, and O, the running sum and the tile's weights not yet consumed are rescaled (rare, exact).
// D: the head dimension, 128 or 64 (one or two 64-wide boxes per tile row).
template <int NQ, bool CAUSAL, bool BF16, int POLY_PERIOD, bool MASKED = false, bool OPTIMISTIC = true, int D = 128>
__device__ __forceinline__ void attention_fwd_kernel(const CUtensorMap* __restrict__ map_q, const CUtensorMap* __restrict__ map_k,
                                                     const CUtensorMap* __restrict__ map_v, void* __restrict__ o_out,
                                                     AttnShape shape, unsigned* status, const float* __restrict__ mask = nullptr) {
    constexpr int BM = 128, BN = 128, UMMA_K = 16, HALVES = D / 64;
    static_assert(D == 64 || D == 128, "head dimension 64 or 128");
    constexpr uint32_t HALF_BYTES = 128 * 64 * 2;          // a 128-row x 64-column 16-bit box: 16 KB
    constexpr uint32_t TILE_BYTES = HALVES * HALF_BYTES;   // 128 x D: 32 KB at D = 128
    constexpr int KV_STAGES = 2;
    constexpr uint32_t TMEM_COLS = 512;
    constexpr uint32_t S_COL = 0, O_COL = 256;  // S_i at i * 128, O_i at 256 + i * 128; P_i over S_i's first 64 columns
    using out_t = typename Half16<BF16>::type;
    static_assert(NQ == 1 || NQ == 2, "one or two query tiles per CTA");

    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* q_smem = smem;                                  // NQ tiles
    uint8_t* k_smem = q_smem + NQ * TILE_BYTES;              // KV_STAGES tiles
    uint8_t* v_smem = k_smem + KV_STAGES * TILE_BYTES;       // KV_STAGES tiles
    uint64_t* bars = reinterpret_cast<uint64_t*>(v_smem + KV_STAGES * TILE_BYTES);
    uint64_t* q_full = bars;                  // 1
    uint64_t* k_full = bars + 1;              // KV_STAGES
    uint64_t* k_empty = k_full + KV_STAGES;
    uint64_t* v_full = k_empty + KV_STAGES;
    uint64_t* v_empty = v_full + KV_STAGES;
    uint64_t* s_full = v_empty + KV_STAGES;   // NQ
    uint64_t* p_ready = s_full + 2;           // NQ
    uint64_t* o_done = p_ready + 2;           // NQ
    uint64_t* p_half = o_done + 2;            // NQ: the first 64 keys of P are written
    uint64_t* o_half = p_half + 2;            // NQ: the first half of P V of a key tile has completed
    uint64_t* q_empty = o_half + 2;           // 1: the item's last Q K^T has read the Q tiles
    uint64_t* item_full = q_empty + 1;        // 2: a work item is published in the ring slot
    uint64_t* item_empty = item_full + 2;     // 2: every role has read it
    uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(item_empty + 2);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);
    volatile int* item_ring = abort_flag + 1;  // 2 slots: item index, or -1 when the work is exhausted
    const tc::Guard guard{status, abort_flag};

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int q_blocks = (shape.seq + NQ * BM - 1) / (NQ * BM);
    const int kv_tiles = (shape.seq + BN - 1) / BN;
    const int num_items = shape.batch_heads * q_blocks;
    unsigned* work_counter = status + 4;  // zero at launch; the last CTA to finish resets it (and status[5])

    // an item: NQ query tiles of one (batch, head); within a head the block with the most keys comes first
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
        tc::mbar_init(q_empty, 1);
        for (int s = 0; s < KV_STAGES; ++s) {
            tc::mbar_init(&k_full[s], 1);
            tc::mbar_init(&k_empty[s], 1);
            tc::mbar_init(&v_full[s], 1);
            tc::mbar_init(&v_empty[s], 1);
        }
        for (int i = 0; i < 2; ++i) {
            tc::mbar_init(&s_full[i], 1);
            tc::mbar_init(&p_ready[i], 4);  // one arrival per softmax warp
            tc::mbar_init(&p_half[i], 4);
            tc::mbar_init(&o_half[i], 1);
            tc::mbar_init(&o_done[i], 1);
            tc::mbar_init(&item_full[i], 1);
            tc::mbar_init(&item_empty[i], 1 + 4 * NQ);  // the MMA thread and every softmax warp
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
            uint32_t kvc = 0;  // K/V tiles loaded so far, over all items: stage and phase come from it
            for (uint32_t it = 0;; ++it) {
                const uint32_t slot = it & 1;
                if (!tc::mbar_wait(&item_empty[slot], ((it >> 1) & 1) ^ 1, guard, tc::WAIT_OTHER, it)) break;
                const unsigned claimed = atomicAdd(work_counter, 1u);
                const int w = claimed < static_cast<unsigned>(num_items) ? static_cast<int>(claimed) : -1;
                item_ring[slot] = w;
                tc::mbar_arrive(&item_full[slot]);  // (release: the slot's value is visible to who sees the phase)
                if (w < 0) break;
                const Item item = decode(w);
                bool alive = true;
                for (int j = 0; alive && j < item.n_max; ++j, ++kvc) {
                    const uint32_t s = kvc % KV_STAGES, ph = (kvc / KV_STAGES) & 1;
                    if (!tc::mbar_wait(&k_empty[s], ph ^ 1, guard, tc::WAIT_SMEM_EMPTY, j)) { alive = false; break; }
                    tc::mbar_arrive_expect_tx(&k_full[s], TILE_BYTES);
#pragma unroll
                    for (int h = 0; h < HALVES; ++h)
                        tc::tma_load_3d(k_smem + s * TILE_BYTES + h * HALF_BYTES, map_k, &k_full[s], h * 64, j * BN, item.bh);
                    if (!tc::mbar_wait(&v_empty[s], ph ^ 1, guard, tc::WAIT_SMEM_EMPTY, 1000 + j)) { alive = false; break; }
                    tc::mbar_arrive_expect_tx(&v_full[s], TILE_BYTES);
#pragma unroll
                    for (int h = 0; h < HALVES; ++h)
                        tc::tma_load_3d(v_smem + s * TILE_BYTES + h * HALF_BYTES, map_v, &v_full[s], h * 64, j * BN, item.bh);
                    if (j == 0) {  // Q after the first K and V: its buffer frees last (the previous item's last Q K^T)
                        if (!tc::mbar_wait(q_empty, (it & 1) ^ 1, guard, tc::WAIT_SMEM_EMPTY, 9000)) { alive = false; break; }
                        tc::mbar_arrive_expect_tx(q_full, NQ * TILE_BYTES);
#pragma unroll
                        for (int i = 0; i < NQ; ++i)
#pragma unroll
                            for (int h = 0; h < HALVES; ++h)
                                tc::tma_load_3d(q_smem + i * TILE_BYTES + h * HALF_BYTES, map_q, q_full, h * 64, item.q0 + i * BM, item.bh);
                    }
                }
                if (!alive) break;
            }
        }
    } else if (warp == 1) {
        // ---------------------------------------------------------------- MMA issuer
        if (tc::elect_one()) {
            constexpr uint32_t idesc_qk = tc::idesc_f16(BM, BN, BF16);
            constexpr uint32_t idesc_pv = tc::idesc_f16(BM, D, BF16) | (1u << 16);  // B (= V) is MN-major
            uint32_t kvc = 0;          // K/V tiles of the items before this one
            uint32_t c[2] = {0, 0};    // key tiles processed per query tile, over all items: the phase of s_full, p_*, o_done
            bool alive = true;
            for (uint32_t it = 0; alive; ++it) {
                const uint32_t slot = it & 1;
                if (!tc::mbar_wait(&item_full[slot], (it >> 1) & 1, guard, tc::WAIT_OTHER, 100 + it)) break;
                const int w = item_ring[slot];
                tc::mbar_arrive(&item_empty[slot]);
                if (w < 0) break;
                const Item item = decode(w);
                if (!tc::mbar_wait(q_full, it & 1, guard, tc::WAIT_SMEM_FULL, 9999)) break;
                int k_waited = -1, v_waited = -1;

                // S_i = Q_i K_j^T: K runs over d = 128 in two 64-wide halves of four 16-wide steps
                auto issue_qk = [&](int i, int j) {
                    const uint32_t t = kvc + j, s = t % KV_STAGES;
                    if (k_waited != j) {
                        if (!tc::mbar_wait(&k_full[s], (t / KV_STAGES) & 1, guard, tc::WAIT_SMEM_FULL, j)) return false;
                        k_waited = j;
                    }
                    tc::tc_fence_after_sync();
                    const uint8_t* qt = q_smem + i * TILE_BYTES;
                    const uint8_t* kt = k_smem + s * TILE_BYTES;
#pragma unroll
                    for (int kk = 0; kk < D / UMMA_K; ++kk) {
                        const uint32_t off = (kk / 4) * HALF_BYTES + (kk % 4) * (UMMA_K * 2);
                        tc::mma_f16_ss(tmem_base + S_COL + i * BN, tc::smem_desc_k128(qt + off), tc::smem_desc_k128(kt + off),
                                       idesc_qk, kk != 0);
                    }
                    tc::mma_commit(&s_full[i]);
                    if (i == NQ - 1) {
                        tc::mma_commit(&k_empty[s]);                      // the last query tile to use K_j
                        if (j == item.n_max - 1) tc::mma_commit(q_empty);  // and the item's last use of Q
                    }
                    return true;
                };
                // O_i += P_i V_j, one 64-key half: V_j is [key][d], d contiguous: MN-major, 64-wide d halves 16 KB
                // apart (leading offset), 8-key groups 1024 B apart (stride offset)
                auto issue_pv = [&](int i, int j, int half) {
                    const uint32_t t = kvc + j, s = t % KV_STAGES;
                    if (v_waited != j) {
                        if (!tc::mbar_wait(&v_full[s], (t / KV_STAGES) & 1, guard, tc::WAIT_SMEM_FULL, 1000 + j)) return false;
                        v_waited = j;
                    }
                    tc::tc_fence_after_sync();
                    const uint8_t* vt = v_smem + s * TILE_BYTES;
#pragma unroll
                    for (int kk = half * 4; kk < half * 4 + 4; ++kk) {
                        uint64_t d = 0;
                        d |= static_cast<uint64_t>((tc::smem_u32(vt + kk * UMMA_K * 128) & 0x3ffff) >> 4);
                        d |= static_cast<uint64_t>(HALF_BYTES >> 4) << 16;  // leading byte offset: next 64 columns of d
                        d |= static_cast<uint64_t>(1024 >> 4) << 32;        // stride byte offset: next 8 keys
                        d |= static_cast<uint64_t>(1) << 46;
                        d |= static_cast<uint64_t>(2) << 61;                // SWIZZLE_128B
                        tc::mma_f16_ts(tmem_base + O_COL + i * D, tmem_base + S_COL + i * BN + kk * (UMMA_K / 2), d, idesc_pv,
                                       (j | kk) != 0);
                    }
                    if (half == 1) {
                        tc::mma_commit(&o_done[i]);
                        if (i == NQ - 1) tc::mma_commit(&v_empty[s]);
                    } else if (OPTIMISTIC) {
                        tc::mma_commit(&o_half[i]);
                    }
                    return true;
                };

#pragma unroll
                for (int i = 0; i < NQ && alive; ++i) alive = issue_qk(i, 0);
                for (int j = 0; alive && j < item.n_max; ++j) {
#pragma unroll
                    for (int i = 0; i < NQ; ++i) {
                        if (!alive || j >= item.n_kv[i]) continue;
                        if (!tc::mbar_wait(&p_half[i], c[i] & 1, guard, tc::WAIT_TMEM_FULL, 2000 + j)) { alive = false; break; }
                        alive = issue_pv(i, j, 0);
                        if (!alive || !tc::mbar_wait(&p_ready[i], c[i] & 1, guard, tc::WAIT_TMEM_FULL, 2500 + j)) { alive = false; break; }
                        alive = issue_pv(i, j, 1);
                        if (alive && j + 1 < item.n_kv[i]) alive = issue_qk(i, j + 1);
                        ++c[i];
                    }
                }
                kvc += item.n_max;
            }
        }
    } else {
        // ---------------------------------------------------------------- softmax, correction, epilogue
        const int i = (warp - 2) >> 2;       // query tile of this warp group
        const int quarter = warp & 3;        // the TMEM lanes this warp may touch: 32 * quarter ..
        const int row = quarter * 32 + lane; // row of the query tile
        const uint32_t lane_addr = static_cast<uint32_t>(quarter * 32) << 16;
        const uint32_t s_addr = tmem_base + lane_addr + S_COL + i * BN;
        const uint32_t o_addr = tmem_base + lane_addr + O_COL + i * D;
        uint32_t steps = 0;  // key tiles this query tile has processed, over all items
        bool alive = i < NQ;
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
            float carried_max = -__int_as_float(0x7f800000);  // the previous tile's row maximum (raw score), not yet in m_used
            for (int j = 0; alive && j < n_mine; ++j, ++steps) {
                if (!tc::mbar_wait(&s_full[i], steps & 1, guard, tc::WAIT_TMEM_FULL, 3000 + j)) {
                    alive = false;
                    break;
                }
                tc::tc_fence_after_sync();
                // keys beyond the query (causal) or beyond the end of the head (a partial last tile) score -inf: on such a
                // tile only columns <= limit are visible
                const int past_end = shape.seq - 1 - j * BN;
                const bool diagonal = (CAUSAL && j == n_mine - 1) || past_end < BN - 1;
                const int limit = CAUSAL ? min(q_row - j * BN, past_end) : past_end;
                uint32_t sr[2][32];                               // two chunks of 32 scores: one in use, one in flight
                // with a mask: score + mask / scale here, so that (score * scale + mask) comes out of the scaling below
                auto add_mask = [&](uint32_t(&cur)[32], int c) {
                    if (MASKED) {
#pragma unroll
                        for (int x = 0; x < 32; ++x) {
                            const int key = min(j * BN + c * 32 + x, shape.seq - 1);
                            cur[x] = __float_as_uint(fmaf(__ldg(mask + key), shape.inv_scale, __uint_as_float(cur[x])));
                        }
                    }
                };
                // O's row times alpha, in tensor memory (every lane of the warp takes part: the accesses are warp-wide)
                auto rescale_o = [&](float alpha) {
#pragma unroll 1
                    for (int c = 0; c < D / 32; ++c) {
                        uint32_t orow[32];
                        tc::tmem_ld_32x32(o_addr + c * 32, orow);
                        tc::tmem_ld_wait();
#pragma unroll
                        for (int x = 0; x < 32; ++x) orow[x] = __float_as_uint(__uint_as_float(orow[x]) * alpha);
                        tc::tmem_st_32x32(o_addr + c * 32, orow);
                    }
                };
                const bool two_pass = !OPTIMISTIC || j == 0;
                float mx = carried_max;
                if (two_pass) {
                    // pass 1: the row maximum (eight independent chains, the next chunk's TMEM load in flight)
                    float mx8[8];
#pragma unroll
                    for (int u = 0; u < 8; ++u) mx8[u] = -__int_as_float(0x7f800000);
                    tc::tmem_ld_32x32(s_addr, sr[0]);
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        tc::tmem_ld_wait();
                        if (c + 1 < 4) tc::tmem_ld_32x32(s_addr + (c + 1) * 32, sr[(c + 1) & 1]);
                        uint32_t(&cur)[32] = sr[c & 1];
                        add_mask(cur, c);
                        if (diagonal) {
#pragma unroll
                            for (int x = 0; x < 32; ++x)
                                if (c * 32 + x > limit) cur[x] = 0xff800000u;
                        }
#pragma unroll
                        for (int x = 0; x < 32; x += 4)
                            mx8[(x / 4) & 7] = emb::max3(mx8[(x / 4) & 7], emb::max3(__uint_as_float(cur[x]), __uint_as_float(cur[x + 1]),
                                                                                     __uint_as_float(cur[x + 2])),
                                                         __uint_as_float(cur[x + 3]));
                    }
                    mx = fmaxf(emb::max3(mx8[0], mx8[1], mx8[2]), emb::max3(emb::max3(mx8[3], mx8[4], mx8[5]), mx8[6], mx8[7]));
                }
                tc::tmem_ld_32x32(s_addr, sr[0]);  // the weights' pass starts: chunk 0, in flight during the bookkeeping
                const float m_new = fmaxf(m_used, mx * shape.scale_log2);
                // move the reference maximum only when it grew by more than 8 (a factor 256): until then the
                // weights are at most 2^8 and the running sum and O stay consistent with the old one
                const bool moved = m_new - m_used > 8.0f;
                if (__any_sync(0xffffffffu, moved) && j > 0) {
                    const float alpha = moved ? emb::ex2_approx_ftz(m_used - m_new) : 1.0f;
                    // PV(i, j-1) completed before S(i, j) did (same issuing thread, in order); the wait orders memory
                    tc::mbar_wait(&o_done[i], (steps - 1) & 1, guard, tc::WAIT_TMEM_EMPTY, 4000 + j);
                    tc::tc_fence_after_sync();
                    rescale_o(alpha);
                    l *= alpha;
                }
                if (moved) m_used = m_new;
                carried_max = -__int_as_float(0x7f800000);
                // pass 2: weights 2^(s * scale - m), their sum, and P as 16-bit pairs over S's own columns
                // (chunk c of P lands on columns 16c .. 16c+15, all of them scores already consumed)
                unsigned long long neg_m2 = emb::pack_f2(-m_used, -m_used);
                const unsigned long long scale2 = emb::pack_f2(shape.scale_log2, shape.scale_log2);
                unsigned long long sum2[2] = {emb::pack_f2(0.0f, 0.0f), emb::pack_f2(0.0f, 0.0f)};
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    tc::tmem_ld_wait();
                    if (c + 1 < 4) tc::tmem_ld_32x32(s_addr + (c + 1) * 32, sr[(c + 1) & 1]);
                    uint32_t(&cur)[32] = sr[c & 1];
                    add_mask(cur, c);
                    if (diagonal) {
#pragma unroll
                        for (int x = 0; x < 32; ++x)
                            if (c * 32 + x > limit) cur[x] = 0xff800000u;
                    }
                    if (!two_pass) {
                        // the chunk's maximum, before any of its weights is made
                        float part[8];
#pragma unroll
                        for (int x = 0; x < 32; x += 4)
                            part[x / 4] = fmaxf(emb::max3(__uint_as_float(cur[x]), __uint_as_float(cur[x + 1]), __uint_as_float(cur[x + 2])),
                                                __uint_as_float(cur[x + 3]));
                        const float cm = fmaxf(emb::max3(part[0], part[1], part[2]), emb::max3(emb::max3(part[3], part[4], part[5]), part[6], part[7]));
                        carried_max = fmaxf(carried_max, cm);
                        const bool over = cm * shape.scale_log2 - m_used > 15.0f;  // its weight would not fit 16 bits
                        if (__any_sync(0xffffffffu, over)) {
                            tc::tmem_ld_wait();  // the next chunk's scores, in flight, land in their registers first
                            const float m_now = over ? cm * shape.scale_log2 : m_used;
                            const float alpha = over ? emb::ex2_approx_ftz(m_used - m_now) : 1.0f;
                            // O holds the earlier tiles and, from the third chunk on, this tile's first half of P V
                            if (c >= 2)
                                tc::mbar_wait(&o_half[i], steps & 1, guard, tc::WAIT_TMEM_EMPTY, 4500 + j);
                            else
                                tc::mbar_wait(&o_done[i], (steps - 1) & 1, guard, tc::WAIT_TMEM_EMPTY, 4600 + j);
                            tc::tc_fence_after_sync();
                            rescale_o(alpha);
                            // this tile's weights already written and not yet handed over
                            for (int cc = (c >= 2 ? 2 : 0); cc < c; ++cc) {
                                uint32_t pw[16];
                                tc::tmem_ld_32x16(s_addr + cc * 16, pw);
                                tc::tmem_ld_wait();
#pragma unroll
                                for (int x = 0; x < 16; ++x) {
                                    float lo, hi;
                                    unpack2<BF16>(pw[x], lo, hi);
                                    pw[x] = pack2<BF16>(lo * alpha, hi * alpha);
                                }
                                asm volatile(
                                    "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
                                    "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};" ::"r"(s_addr + cc * 16),
                                    "r"(pw[0]), "r"(pw[1]), "r"(pw[2]), "r"(pw[3]), "r"(pw[4]), "r"(pw[5]), "r"(pw[6]), "r"(pw[7]),
                                    "r"(pw[8]), "r"(pw[9]), "r"(pw[10]), "r"(pw[11]), "r"(pw[12]), "r"(pw[13]), "r"(pw[14]), "r"(pw[15])
                                    : "memory");
                            }
                            tc::tmem_st_wait();
                            const unsigned long long alpha2 = emb::pack_f2(alpha, alpha), zero2 = emb::pack_f2(0.0f, 0.0f);
                            sum2[0] = emb::fma_f2(sum2[0], alpha2, zero2);
                            sum2[1] = emb::fma_f2(sum2[1], alpha2, zero2);
                            l *= alpha;
                            if (over) m_used = m_now;
                            neg_m2 = emb::pack_f2(-m_used, -m_used);
                        }
                    }
                    uint32_t packed[16];
#pragma unroll
                    for (int x = 0; x < 32; x += 2) {
                        const unsigned long long t2 =
                            emb::fma_f2(emb::pack_f2(__uint_as_float(cur[x]), __uint_as_float(cur[x + 1])), scale2, neg_m2);
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
                        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};" ::"r"(s_addr + c * 16),
                        "r"(packed[0]), "r"(packed[1]), "r"(packed[2]), "r"(packed[3]), "r"(packed[4]), "r"(packed[5]),
                        "r"(packed[6]), "r"(packed[7]), "r"(packed[8]), "r"(packed[9]), "r"(packed[10]), "r"(packed[11]),
                        "r"(packed[12]), "r"(packed[13]), "r"(packed[14]), "r"(packed[15])
                        : "memory");
                    if (c == 1) {  // the first 64 keys' weights are in place: their half of P V may start
                        tc::tmem_st_wait();
                        tc::tc_fence_before_sync();
                        __syncwarp();
                        if (lane == 0) tc::mbar_arrive(&p_half[i]);
                    }
                }
                float sum, sum_hi;
                emb::unpack_f2(emb::add_f2(sum2[0], sum2[1]), sum, sum_hi);
                sum += sum_hi;
                l += sum;
                tc::tmem_st_wait();
                tc::tc_fence_before_sync();
                __syncwarp();
                if (lane == 0) tc::mbar_arrive(&p_ready[i]);
            }
            // PV of the item's last key tile is phase steps - 1 of o_done
            if (alive && tc::mbar_wait(&o_done[i], (steps - 1) & 1, guard, tc::WAIT_TMEM_EMPTY, 5000)) {
                tc::tc_fence_after_sync();
                const float inv = 1.0f / l;
                out_t* dst = static_cast<out_t*>(o_out) + (static_cast<size_t>(row_base) + q_row) * D;
#pragma unroll 1
                for (int c = 0; c < D / 32; ++c) {
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
