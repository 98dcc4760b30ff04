// Prefill attention over the paged bfloat16 cache on the fifth-generation tensor cores.
//
// Same job and same arguments as the mma.sync prefill kernel (portions of prompts of any length
// at any offset, causal, grouped-query, optional window; the host lists tiles of 128 query tokens),
// for head sizes 64 and 128 and pages of 8..128 tokens that divide 128.
//
// One CTA handles one tile of 128 query tokens for TWO query heads that share a key/value head,
// so every key/value block it brings into shared memory is used twice.  Ten warps:
//   warps 0-3   softmax of head A: thread r owns query row r (tensor-memory lane r)
//   warps 4-7   softmax of head B
//   warp 8      producer: TMA copies of Q (once) and of the K and V blocks through the block table
//               into a ring of shared-memory slots (five of 32 KB at head size 128).  Pages that lie
//               one after the other in the pool are fetched together: a block of 128 keys whose
//               pages are all consecutive is one copy, otherwise every aligned run of 2, 4, ...
//               consecutive pages is one (a copy of one 16-token page moves 2 KB and costs about as
//               much to issue as one of 32 KB).  Absent pages are fetched at an out-of-range
//               coordinate, which fills zeros.  The block table's entries are read one block ahead
//   warp 9      allocates tensor memory; walks the schedule as a whole warp, one lane issues tcgen05.mma
// Per block of 128 keys (aligned to absolute positions) and per head:
//   S = Q K^T         M 128 x N 128 x K head size; Q and K are K-major tiles in shared memory; S in
//                     tensor memory
//   softmax           each thread reads its row of S with tcgen05.ld, applies the causal/window
//                     limits of its row, takes exponentials in float32 and writes P as bfloat16 back
//                     into tensor memory (tcgen05.st), two values a column, over the first half of
//                     the columns S came from
//   O += P V          M 128 x N head size x K 128; P is the A operand straight from tensor memory,
//                     V is used as stored ([key][dim]: an MN-major tile in shared memory); O
//                     accumulates in tensor memory over all blocks.  The exponentials are taken
//                     against a reference maximum that follows the row's running maximum only when
//                     that has grown by more than 8 (in log2 units); only then is the row of O
//                     rescaled (tcgen05.ld, multiply, tcgen05.st), which after the first blocks is rare
// Shared memory's bandwidth is what this kernel would otherwise run into: a 128 x 128 x 16 product
// with both operands there reads 8 KB in the 64 cycles it takes, all the 128 bytes a cycle an SM has;
// P written to and read back from shared memory came on top of that (and took two 32 KB buffers that
// are now two more slots of the ring).
// The issue order alternates the heads (PV_A(j), QK_A(j+1), PV_B(j), QK_B(j+1)), so that the
// tensor core works for one head while the other head's softmax runs.  Tensor memory's 512 columns
// are full with that (S and O of two heads), so a head's chain softmax -> PV -> QK -> softmax cannot
// be shortened by computing scores ahead.
// A CTA with one head only (steps with few tiles, see launch_prefill_tc) uses what the second head
// leaves free to run ahead of itself instead: scores alternate between two regions of tensor memory
// (each with its probabilities), so S(j+1) = Q K(j+1)^T is computed while the softmax of block j runs
// (only P V waits for the probabilities), and the second head's query buffer is one more slot of the
// K/V ring.  Blocks then follow one another at the softmax's pace.
// Formulas: crates/aien-inference-abi/src/backend.rs:280-306, scale 1/sqrt(head_dim).
//
// Every wait is bounded; one that runs out records a code (aien_attention_prefill_tc_error) and
// the kernel runs on to its end, frees its tensor memory and returns.  The cache must hold finite
// values everywhere (it is zero-initialised and only ever written with activations): whole pages
// are loaded, and a key that is masked still meets a zero weight in P V.
#include "tma.cuh"
#include "umma.cuh"
#include <math.h>

namespace aien {

__device__ __forceinline__ float max3(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}

constexpr int PT_BM = 128, PT_BN = 128, PT_THREADS = 320;
constexpr int PT_SMEM_MAX = 227 * 1024;

template <int HD> struct PtShape {
    static constexpr int CHUNKS = HD / 64;                       // 64-column (128-byte) chunks of a row
    static constexpr int Q_BYTES = PT_BM * HD * 2;               // one head's query tile
    static constexpr int SLOT_BYTES = PT_BN * HD * 2;            // one K or V block
    static constexpr int FIXED = 2 * Q_BYTES + 1024 /*align*/ + 256 /*barriers*/;
    static constexpr int SLOTS_FIT = (PT_SMEM_MAX - FIXED) / SLOT_BYTES;
    static constexpr int SLOTS = SLOTS_FIT > 6 ? 6 : SLOTS_FIT;
    static constexpr int SMEM = FIXED + SLOTS * SLOT_BYTES;
    static_assert(SLOTS >= 3, "the K/V ring needs three slots");
};

__device__ __forceinline__ float ex2_approx(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// The cache seen through boxes of 1, 2, 4, ... pages of rows by 64 columns (m[k]: page_size << k
// rows), and through one box of 128 rows by the whole head (blk; three-dimensional, chunk-major in
// shared memory as the slots are laid out).
struct PtMaps {
    CUtensorMap m[5];
    CUtensorMap blk;
};

template <int HD>
__global__ void __launch_bounds__(PT_THREADS, 1)
prefill_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ PtMaps maps_k,
                  const __grid_constant__ PtMaps maps_v, const int* __restrict__ block_table, int max_blocks,
                  const int* __restrict__ q_start, const int* __restrict__ ctx_len, const int* __restrict__ tile_seq,
                  const int* __restrict__ tile_q0, int num_tiles, __nv_bfloat16* __restrict__ out, long out_stride,
                  int nq, int nkv, int page_size, int window, float scale_log2e, int cache_rows, int heads_per_cta, int big_boxes,
                  int nsplit, float* __restrict__ part_o, float* __restrict__ part_ml) {
    using S = PtShape<HD>;
    extern __shared__ uint8_t pt_smem[];
    const uint32_t base = (smem_u32(pt_smem) + 1023u) & ~1023u;
    const uint32_t sQ = base, sKV = sQ + 2 * S::Q_BYTES;
    const uint32_t bars = sKV + S::SLOTS * S::SLOT_BYTES;
    const uint32_t q_full = bars, kv_full0 = bars + 8, kv_free0 = kv_full0 + 8 * (S::SLOTS + 1);
    const uint32_t s_ready0 = kv_free0 + 8 * (S::SLOTS + 1), p_ready0 = s_ready0 + 16, o_ready0 = p_ready0 + 16;
    const uint32_t tmem_slot = o_ready0 + 16;
    uint8_t* gen = pt_smem + (base - smem_u32(pt_smem));
    volatile uint32_t* tmem_slot_ptr = reinterpret_cast<volatile uint32_t*>(gen + (tmem_slot - base));

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    // ---- which tile, which heads (the last tiles of a request see the most keys: they start first)
    // heads_per_cta 2: two query heads of a kv head share the CTA's K/V blocks; 1: one head per CTA,
    // for steps with so few tiles that the pairs would leave SMs idle
    const int group = nq / nkv, pairs = (group + heads_per_cta - 1) / heads_per_cta;
    const int per_tile = nkv * pairs;
    // nsplit > 1: the key blocks of a tile are cut into nsplit ranges, one CTA each, which leave
    // unnormalised partial results that prefill_merge_splits_kernel adds up (steps with few tiles and
    // long contexts: few long CTAs would leave most SMs idle)
    const int unit = (int)(blockIdx.x / nsplit), split = (int)(blockIdx.x % nsplit);
    const int tile = num_tiles - 1 - unit / per_tile;
    const int rem = unit % per_tile;
    const int kvh = rem / pairs, pair = rem - kvh * pairs;
    const int head_a = kvh * group + heads_per_cta * pair;
    const bool has_b = heads_per_cta == 2 && 2 * pair + 1 < group;
    const int s = tile_seq[tile], q0 = tile_q0[tile];
    const int qs = q_start[s], q_len = q_start[s + 1] - qs;
    const int rows = min(PT_BM, q_len - q0);
    const int pos0 = ctx_len[s] - q_len + q0;                      // position of the tile's first query
    const int pos_last = pos0 + rows - 1;
    const int first = (window > 0 && pos0 - window + 1 > 0) ? pos0 - window + 1 : 0;
    const int kb_first = first / PT_BN, kb_last = pos_last / PT_BN;
    const int per_split = (kb_last - kb_first + nsplit) / nsplit;         // ranges of whole blocks, in order: what a range holds
    const int kb_begin = kb_first + split * per_split;                   // depends on the tile's keys and nsplit alone
    const int kb_end = min(kb_last, kb_begin + per_split - 1);
    const int nb = kb_end - kb_begin + 1;                                // <= 0: nothing in this range

    griddep_launch();
    if (threadIdx.x == 0) {
        mbar_init(q_full, 1);
        for (int i = 0; i < S::SLOTS + 1; ++i) { mbar_init(kv_full0 + 8 * i, 1); mbar_init(kv_free0 + 8 * i, 1); }
        for (int h = 0; h < 2; ++h) { mbar_init(s_ready0 + 8 * h, 1); mbar_init(p_ready0 + 8 * h, 128); mbar_init(o_ready0 + 8 * h, 1); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 9) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tmem_slot), "r"(512u) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = *tmem_slot_ptr;
    // tensor-memory columns: S of head A, S of head B, then the outputs O of A and of B
    const uint32_t tS0 = tmem, tO0 = tmem + 2 * PT_BN;
    // one head alone: the other head's query buffer serves as one more slot of the K/V ring
    const bool single = !has_b;
    constexpr int NS1 = S::SLOTS + 1;                   // ring slots of a CTA with one head
    auto slot_addr = [&](int slot) { return slot < S::SLOTS ? sKV + slot * S::SLOT_BYTES : sQ + S::Q_BYTES; };

    if (nb <= 0) {
        // an empty range: weight zero in the merge
        if (warp < 8 && (warp < 4 || has_b)) {
            const int h = warp >> 2, r = (warp & 3) * 32 + lane;
            float* ml = part_ml + ((((size_t)tile * PT_BM + r) * nq + head_a + h) * nsplit + split) * 2;
            ml[0] = -INFINITY;
            ml[1] = 0.f;
        }
    } else if (warp == 8) {
        // ------------------------------------------------------------------ producer
        const int pages_per_block = PT_BN / page_size;
        const int* bt = block_table + (size_t)s * max_blocks;
        auto item_is_v = [&](int item) { return single ? (item >= 2 && (item & 1) == 0) || item == 2 * nb - 1 : (bool)(item & 1); };
        auto item_block = [&](int item) {
            return kb_begin + (single ? (item_is_v(item) ? (item == 2 * nb - 1 ? nb - 1 : item / 2 - 1) : (item + 1) / 2) : (item >> 1));
        };
        // this lane's page of a key block (-1: none); asked for one item ahead, so that the table's
        // latency passes under the wait for a free slot
        auto page_of = [&](int kb) {
            int page = -1;
            if (lane < pages_per_block) {
                const int key0 = kb * PT_BN + lane * page_size;
                const int blk = key0 / page_size;
                if (key0 <= pos_last && key0 + page_size > first && blk < max_blocks) page = bt[blk];
            }
            return page;
        };
        int page_next = page_of(item_block(0));          // the table is this step's metadata, not the work of the kernel ahead
        // Queries and this step's rows of the caches come from the kernel ahead in the stream: with a
        // dependent launch everything above ran beside its tail, and no other warp touches global
        // memory before it has data from this one.
        griddep_wait();
        if (lane == 0) {
            mbar_expect_tx(q_full, (has_b ? 2 : 1) * S::Q_BYTES);
            for (int h = 0; h < (has_b ? 2 : 1); ++h)
                for (int c = 0; c < S::CHUNKS; ++c)
                    tma_load_2d(sQ + h * S::Q_BYTES + c * (PT_BM * 128), &map_q, q_full, (head_a + h) * HD + c * 64, qs + q0);
        }
        for (int item = 0; item < 2 * nb; ++item) {                 // K0 V0 K1 V1 ...; one head alone: K0 K1 V0 K2 V1 ...
            const int slot = single ? item % NS1 : item % S::SLOTS;
            const int round = single ? item / NS1 : item / S::SLOTS;
            const int page = page_next;
            if (item + 1 < 2 * nb) page_next = page_of(item_block(item + 1));
            if (round > 0) mbar_wait(kv_free0 + 8 * slot, (round - 1) & 1, 1);
            const bool is_v = item_is_v(item);
            if (lane == 0) mbar_expect_tx(kv_full0 + 8 * slot, S::SLOT_BYTES);
            __syncwarp();
            // lane i's page continues lane i-1's in the pool; the largest aligned group of 2, 4, ... pages
            // around this lane whose pages all continue one another is fetched by its first lane
            const int prev = __shfl_up_sync(0xffffffffu, page, 1);
            const uint32_t links = __ballot_sync(0xffffffffu, lane > 0 && lane < pages_per_block && page >= 0 && prev >= 0 && page == prev + 1);
            int g = 1, level = 0;
            for (int gg = 2, lv = 1; gg <= pages_per_block; gg <<= 1, ++lv) {
                const int a = lane & ~(gg - 1);
                const uint32_t need = (((gg >= 32 ? 0u : (1u << gg)) - 1u) << a) & ~(1u << a);
                if ((links & need) != need) break;
                g = gg; level = lv;
            }
            if (lane < pages_per_block && (lane & (g - 1)) == 0) {
                const int row = page >= 0 ? page * page_size : cache_rows;     // out of range: zeros
                const PtMaps& maps = is_v ? maps_v : maps_k;
                const uint32_t dst = slot_addr(slot) + lane * page_size * 128;
                if (g == pages_per_block && big_boxes) {
                    tma_load_3d(dst, &maps.blk, kv_full0 + 8 * slot, 0, row, kvh * S::CHUNKS);      // the whole block in one copy
                } else {
                    for (int c = 0; c < S::CHUNKS; ++c)
                        tma_load_2d(dst + c * (PT_BN * 128), &maps.m[level], kv_full0 + 8 * slot, kvh * HD + c * 64, row);
                }
            }
        }
    } else if (warp == 9) {
        // ------------------------------------------------------------------ MMA issue
        // The whole warp walks the schedule and waits on the barriers, so that addresses and descriptors
        // are the same in every lane (and cheap to form); one lane issues.
        {
            const bool issuer = lane == 0;
            const uint32_t idesc_qk = umma_idesc_bf16(PT_BM, PT_BN, false);
            const uint32_t idesc_pv = umma_idesc_bf16(PT_BM, HD, true);
            const uint64_t desc_q0 = make_desc_sw128(sQ);
            // S[region] = Q(head) K^T from the K block in the slot at `b`
            auto qk = [&](int head, int region, uint32_t b, uint32_t bar) {
                const uint64_t da = desc_q0 + (uint64_t)((head * S::Q_BYTES) >> 4), db = make_desc_sw128(b);
                if (issuer) {
#pragma unroll
                    for (int kk = 0; kk < HD / 16; ++kk) {
                        const uint64_t off = (uint64_t)(((kk >> 2) * (PT_BM * 128) + (kk & 3) * 32) >> 4);
                        umma_bf16(tS0 + region * PT_BN, da + off, db + off, idesc_qk, kk > 0 ? 1u : 0u);
                    }
                    umma_commit(bar);
                }
            };
            // O[head] += P V: P from the first 64 columns of score region `region`, V from the slot at `b`
            auto pv = [&](int head, int region, uint32_t b, bool first_block, uint32_t bar) {
                const uint64_t db = make_desc_sw128_mn(b, PT_BN * 128);
                if (issuer) {
#pragma unroll
                    for (int kk = 0; kk < PT_BN / 16; ++kk)
                        umma_bf16_ts(tO0 + head * HD, tS0 + region * PT_BN + kk * 8, db + (uint64_t)((kk * 16 * 128) >> 4), idesc_pv, (kk > 0 || !first_block) ? 1u : 0u);
                    umma_commit(bar);
                }
            };
            auto commit = [&](uint32_t bar) { if (issuer) umma_commit(bar); };
            // (data that TMA wrote is visible to the tensor core once the barrier has completed)
            auto wait_item = [&](int item) { mbar_wait(kv_full0 + 8 * (item % S::SLOTS), (item / S::SLOTS) & 1, 2); };
            auto wait_item1 = [&](int item) { mbar_wait(kv_full0 + 8 * (item % NS1), (item / NS1) & 1, 2); };   // the ring of a CTA with one head
            mbar_wait(q_full, 0, 3);
            if (single) {
                // One head: scores of block j go to region j & 1 of tensor memory (and its probabilities
                // back into that region), and the items come in the order they are used: K0 K1 V0 K2 V1 K3 ...
                int item = 0;
                wait_item1(item); qk(0, 0, slot_addr(item % NS1), s_ready0); commit(kv_free0 + 8 * (item % NS1)); ++item;
                if (nb > 1) { wait_item1(item); qk(0, 1, slot_addr(item % NS1), s_ready0 + 8); commit(kv_free0 + 8 * (item % NS1)); ++item; }
                for (int j = 0; j < nb; ++j) {
                    const int buf = j & 1;
                    wait_item1(item);
                    mbar_wait(p_ready0 + 8 * buf, (j >> 1) & 1, 4);          // P[buf] is written
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    pv(0, buf, slot_addr(item % NS1), j == 0, o_ready0);
                    commit(kv_free0 + 8 * (item % NS1));
                    ++item;
                    if (j + 2 < nb) { wait_item1(item); qk(0, buf, slot_addr(item % NS1), s_ready0 + 8 * buf); commit(kv_free0 + 8 * (item % NS1)); ++item; }
                }
            } else {
                wait_item(0);
                qk(0, 0, sKV, s_ready0);
                if (has_b) qk(1, 1, sKV, s_ready0 + 8);
                commit(kv_free0);
                for (int j = 0; j < nb; ++j) {
                    const int v_item = 2 * j + 1, k_item = 2 * j + 2;
                    const bool more = j + 1 < nb;
                    const uint32_t v_at = sKV + (v_item % S::SLOTS) * S::SLOT_BYTES, k_at = sKV + (k_item % S::SLOTS) * S::SLOT_BYTES;
                    // the blocks themselves have long arrived: seen to before the probabilities are awaited
                    wait_item(v_item);
                    if (more) wait_item(k_item);
                    mbar_wait(p_ready0, j & 1, 4);
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    pv(0, 0, v_at, j == 0, o_ready0);
                    if (more) qk(0, 0, k_at, s_ready0);
                    if (has_b) {
                        mbar_wait(p_ready0 + 8, j & 1, 5);
                        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                        pv(1, 1, v_at, j == 0, o_ready0 + 8);
                    }
                    commit(kv_free0 + 8 * (v_item % S::SLOTS));
                    if (more) {
                        if (has_b) qk(1, 1, k_at, s_ready0 + 8);
                        commit(kv_free0 + 8 * (k_item % S::SLOTS));
                    }
                }
            }
        }
    } else if (warp < 4 || has_b) {
        // ------------------------------------------------------------------ softmax
        const int h = warp >> 2, quarter = warp & 3;
        const int r = quarter * 32 + lane;
        const uint32_t lane_off = (uint32_t)(quarter * 32) << 16;
        // one head alone alternates between two score regions and two probability buffers (h is 0 then)
        const uint32_t tS_base = tS0 + h * PT_BN + lane_off, tO = tO0 + h * HD + lane_off;
        const int hi = r < rows ? pos0 + r : -1;                                 // last key this row sees
        const int lo = (window > 0 && hi - window + 1 > 0) ? hi - window + 1 : 0;
        // m_ref: the maximum the exponentials are taken against.  It follows the row's running
        // maximum only when that has grown by more than 8 (a factor 256, harmless in float32 and
        // in bfloat16's exponent), so the output in tensor memory is rescaled rarely.
        float m_ref = -INFINITY, l_run = 0.f;

        for (int j = 0; j < nb; ++j) {
            const int key_base = (kb_begin + j) * PT_BN;
            const int buf = single ? (j & 1) : 0;
            const uint32_t tS = tS_base + buf * PT_BN;
            mbar_wait(s_ready0 + 8 * (single ? buf : h), (single ? (j >> 1) : j) & 1, 6);
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            uint32_t v[PT_BN];
#pragma unroll
            for (int c0 = 0; c0 < PT_BN; c0 += 32) tmem_ld32(tS + c0, v + c0);
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
            if (key_base + PT_BN - 1 > hi) {                                     // the block on the diagonal: columns beyond hi
                const int last = hi - key_base;
#pragma unroll
                for (int i = 0; i < PT_BN; ++i)
                    if (i > last) v[i] = 0xff800000u;                            // -inf
            }
            if (key_base < lo) {                                                 // the window's far edge
                const int first_col = lo - key_base;
#pragma unroll
                for (int i = 0; i < PT_BN; ++i)
                    if (i < first_col) v[i] = 0xff800000u;
            }
            float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};           // four chains: the instruction's latency, not its rate, would bound one
#pragma unroll
            for (int i = 0; i < PT_BN; i += 8) {
#pragma unroll
                for (int c = 0; c < 4; ++c) mx4[c] = max3(mx4[c], __uint_as_float(v[i + 2 * c]), __uint_as_float(v[i + 2 * c + 1]));
            }
            float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
            mx *= scale_log2e;
            if (j == 0) {
                m_ref = mx;
            } else {
                const bool grow = mx > m_ref + 8.0f;
                if (__any_sync(0xffffffffu, grow)) {
                    // the block product of j-1 must have landed before the output is touched
                    mbar_wait(o_ready0 + 8 * h, (j - 1) & 1, 7);
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    float f = 1.0f;
                    if (grow) {
                        f = (m_ref == -INFINITY) ? 0.f : ex2_approx(m_ref - mx);
                        m_ref = mx;
                        l_run *= f;
                    }
#pragma unroll 1
                    for (int c0 = 0; c0 < HD; c0 += 32) {
                        uint32_t o[32];
                        tmem_ld32(tO + c0, o);
                        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                        for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * f);
                        tmem_st32(tO + c0, o);
                    }
                    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
                }
            }
            const float neg_base = (m_ref == -INFINITY) ? 0.f : -m_ref;
            // The probabilities go back to tensor memory as bfloat16, two a column, over the first half
            // of the columns the scores came from (all of which this thread has read): the block product
            // takes them from there as its A operand.  The tensor core runs its products in the order
            // they were issued, so the score product that next writes these columns comes after it.
            float sum = 0.f;
#pragma unroll
            for (int c0 = 0; c0 < PT_BN; c0 += 64) {
                uint32_t pk[32];
#pragma unroll
                for (int i = 0; i < 32; ++i) {
                    const float p0 = ex2_approx(fmaf(__uint_as_float(v[c0 + 2 * i]), scale_log2e, neg_base));      // exp2(-inf) = 0 for masked keys
                    const float p1 = ex2_approx(fmaf(__uint_as_float(v[c0 + 2 * i + 1]), scale_log2e, neg_base));
                    sum += p0 + p1;
                    __nv_bfloat162 pp = __floats2bfloat162_rn(p0, p1);
                    pk[i] = *reinterpret_cast<uint32_t*>(&pp);
                }
                tmem_st32(tS + (c0 >> 1), pk);
            }
            l_run += sum;
            asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
            // One head alone: the scores of this block were issued behind the block product of two blocks
            // ago, not of the last one, so they do not tell that that one has landed.  A wait names a
            // phase by its parity, which is only right while at most one phase can have completed unseen:
            // every product is therefore seen off here, one block late (it has long landed), before this
            // thread's hand-over lets the next one be issued.  The waits on o_ready above and at the end
            // rely on it.
            if (single && j > 0) mbar_wait(o_ready0, (j - 1) & 1, 7);
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            mbar_arrive(p_ready0 + 8 * (single ? buf : h));
        }

        mbar_wait(o_ready0 + 8 * h, (nb - 1) & 1, 7);
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        if (nsplit > 1) {
            // this range's part: the unnormalised sums, the maximum they are taken against (log2 units) and the weight sum
            const size_t prow = (((size_t)tile * PT_BM + r) * nq + head_a + h) * nsplit + split;
            part_ml[prow * 2] = m_ref;
            part_ml[prow * 2 + 1] = l_run;
            float* dstf = part_o + prow * HD;
#pragma unroll 1
            for (int c0 = 0; c0 < HD; c0 += 32) {
                uint32_t o[32];
                tmem_ld32(tO + c0, o);
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                for (int d = 0; d < 32; d += 4)
                    *reinterpret_cast<uint4*>(dstf + c0 + d) = make_uint4(o[d], o[d + 1], o[d + 2], o[d + 3]);
            }
        } else {
        const float inv = l_run > 0.f ? 1.0f / l_run : 0.f;
        __nv_bfloat16* dst = out + (size_t)(qs + q0 + (r < rows ? r : 0)) * out_stride + (size_t)(head_a + h) * HD;
#pragma unroll 1
        for (int c0 = 0; c0 < HD; c0 += 32) {
            uint32_t o[32];
            tmem_ld32(tO + c0, o);
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
            if (r < rows) {
#pragma unroll
                for (int d = 0; d < 32; d += 8) {
                    __nv_bfloat162 a = __floats2bfloat162_rn(__uint_as_float(o[d]) * inv, __uint_as_float(o[d + 1]) * inv);
                    __nv_bfloat162 b = __floats2bfloat162_rn(__uint_as_float(o[d + 2]) * inv, __uint_as_float(o[d + 3]) * inv);
                    __nv_bfloat162 c = __floats2bfloat162_rn(__uint_as_float(o[d + 4]) * inv, __uint_as_float(o[d + 5]) * inv);
                    __nv_bfloat162 e = __floats2bfloat162_rn(__uint_as_float(o[d + 6]) * inv, __uint_as_float(o[d + 7]) * inv);
                    uint4 w;
                    w.x = *reinterpret_cast<uint32_t*>(&a); w.y = *reinterpret_cast<uint32_t*>(&b);
                    w.z = *reinterpret_cast<uint32_t*>(&c); w.w = *reinterpret_cast<uint32_t*>(&e);
                    *reinterpret_cast<uint4*>(dst + c0 + d) = w;
                }
            }
        }
        }
    }

    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 9) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512u) : "memory");
    }
}

// Adds up the parts that the key ranges of a tile left: out = sum_s w_s O_s / sum_s w_s l_s with
// w_s = 2^(m_s - max m), in the order of the ranges.  One warp per (query row, head), a lane per
// HD / 32 dimensions; all loads of a warp are independent of one another.
constexpr int PT_MAX_SPLITS = 8;
template <int HD>
__global__ void __launch_bounds__(256) prefill_merge_splits_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                                                   const int* __restrict__ q_start, const int* __restrict__ tile_seq,
                                                                   const int* __restrict__ tile_q0, __nv_bfloat16* __restrict__ out,
                                                                   long out_stride, int nq, int nsplit) {
    constexpr int PER = HD / 32;
    griddep_launch();
    const int lane = threadIdx.x & 31;
    const long unit = (long)blockIdx.x * 8 + (threadIdx.x >> 5);          // (tile, row, head)
    const int head = (int)(unit % nq);
    const long trow = unit / nq;
    const int tile = (int)(trow / PT_BM), r = (int)(trow % PT_BM);
    const int s = tile_seq[tile], q0 = tile_q0[tile];
    const int qs = q_start[s], q_len = q_start[s + 1] - qs;
    griddep_wait();
    if (r >= min(PT_BM, q_len - q0)) return;
    const size_t prow = (size_t)unit * nsplit;
    float m[PT_MAX_SPLITS], l[PT_MAX_SPLITS], o[PT_MAX_SPLITS][PER];
#pragma unroll
    for (int sp = 0; sp < PT_MAX_SPLITS; ++sp) {
        m[sp] = -INFINITY; l[sp] = 0.f;
        if (sp < nsplit) { m[sp] = __ldcg(part_ml + (prow + sp) * 2); l[sp] = __ldcg(part_ml + (prow + sp) * 2 + 1); }
    }
#pragma unroll
    for (int sp = 0; sp < PT_MAX_SPLITS; ++sp) {
        const bool live = sp < nsplit && m[sp] != -INFINITY && l[sp] > 0.f;    // an empty range left no sums
        if (!live) m[sp] = -INFINITY;
        const float* src = part_o + (prow + sp) * HD + lane * PER;
        if constexpr (PER == 4) {
            const float4 t = live ? __ldcg(reinterpret_cast<const float4*>(src)) : make_float4(0.f, 0.f, 0.f, 0.f);
            o[sp][0] = t.x; o[sp][1] = t.y; o[sp][2] = t.z; o[sp][3] = t.w;
        } else {
            const float2 t = live ? __ldcg(reinterpret_cast<const float2*>(src)) : make_float2(0.f, 0.f);
            o[sp][0] = t.x; o[sp][1] = t.y;
        }
    }
    float M = -INFINITY;
#pragma unroll
    for (int sp = 0; sp < PT_MAX_SPLITS; ++sp) M = fmaxf(M, m[sp]);
    float L = 0.f, acc[PER];
#pragma unroll
    for (int i = 0; i < PER; ++i) acc[i] = 0.f;
#pragma unroll
    for (int sp = 0; sp < PT_MAX_SPLITS; ++sp) {
        const float w = m[sp] == -INFINITY ? 0.f : ex2_approx(m[sp] - M);
        L = fmaf(w, l[sp], L);
#pragma unroll
        for (int i = 0; i < PER; ++i) acc[i] = fmaf(w, o[sp][i], acc[i]);
    }
    const float inv = L > 0.f ? 1.0f / L : 0.f;
    __nv_bfloat16* dst = out + (size_t)(qs + q0 + r) * out_stride + (size_t)head * HD + lane * PER;
#pragma unroll
    for (int i = 0; i < PER; i += 2) *reinterpret_cast<__nv_bfloat162*>(dst + i) = __floats2bfloat162_rn(acc[i] * inv, acc[i + 1] * inv);
}

template <int HD>
static int launch_prefill_tc(const CUtensorMap& mq, const PtMaps& mk, const PtMaps& mv, int big_boxes, const int* bt, int max_blocks,
                             const int* q_start, const int* ctx_len, const int* tile_seq, const int* tile_q0, int num_tiles,
                             void* out, long out_stride, int nq, int nkv, int page_size, int window, float scale, int cache_rows,
                             void* scratch, long scratch_bytes, int max_ctx, int force_splits, cudaStream_t stream) {
    auto kern = prefill_tc_kernel<HD>;
    static bool configured = false;
    if (!configured) {
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, PtShape<HD>::SMEM) != cudaSuccess) return AIEN_E_STATE;
        configured = true;
    }
    const int group = nq / nkv;
    int sms = 148, dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) sms = 148;
    // Two heads of a kv head per CTA halve the K/V traffic and let the tensor core work for one head
    // under the other's softmax: a key block then takes ~3,550 cycles for both heads, against ~2,870 for
    // the single head of a CTA that has only one (and runs its score products ahead); a CTA costs
    // ~6,000 cycles beside its blocks.  What decides is the number of waves either way: 512 tokens are
    // 128 single-head CTAs, one wave, against 64 pairs that leave half the SMs idle.
    // Few tiles over long contexts (a portion at the end of a long prompt) can do better than either:
    // pairs, with the keys of every tile cut into ranges on separate CTAs, at the price of the partial
    // results' way through memory and of the merge: ~20,000 cycles when timed alone, counted double
    // here because inside a step the partial results also push weights out of L2 (a 512-token portion
    // at offset 2,048 beside 24 decoding requests: equal alone, 0.4 ms a step slower with two ranges).
    // Measured (32 / 8 heads of 128): 256 tokens at offset 7,936 110 -> 50 us (4 ranges), 128 at 4,000
    // 59 -> 26 us (8); 512 tokens at 3,584 would gain little (58 -> 51 us alone) and are left alone.
    const long single = (long)num_tiles * nkv * group, paired = (long)num_tiles * nkv * ((group + 1) / 2);
    auto waves = [&](long ctas) { return (ctas + sms - 1) / sms; };
    const long blocks = max_ctx > 0 ? (max_ctx + PT_BN - 1) / PT_BN : 0;          // of the longest tile, at most
    int heads_per_cta = (group >= 2 && 18 * waves(single) > 25 * waves(paired)) ? 2 : 1;
    int nsplit = 1;
    const long part_rows = (long)num_tiles * PT_BM * nq;
    auto fits = [&](int n) { return scratch != nullptr && part_rows * n * (HD + 2) * 4 <= scratch_bytes; };
    if (force_splits > 0) {
        nsplit = force_splits;
        if (!fits(nsplit)) return AIEN_E_SHAPE;
    } else if (group >= 2 && blocks > 0) {
        long best = heads_per_cta == 2 ? waves(paired) * (blocks * 3550 + 6000) : waves(single) * (blocks * 2870 + 6000);
        for (int n = 2; n <= PT_MAX_SPLITS && fits(n); ++n) {
            const long t = waves(paired * n) * ((blocks + n - 1) / n * 3550 + 6000) + 40000;
            if (t < best) { best = t; nsplit = n; }
        }
    }
    if (nsplit > 1 && group >= 2) heads_per_cta = 2;
    const long ctas = (long)num_tiles * nkv * ((group + heads_per_cta - 1) / heads_per_cta) * nsplit;
    if (ctas > 2147483647L) return AIEN_E_SHAPE;
    float* part_o = nsplit > 1 ? (float*)scratch : nullptr;
    float* part_ml = nsplit > 1 ? part_o + part_rows * nsplit * HD : nullptr;
    launch_chain(kern, dim3((unsigned)ctas), dim3(PT_THREADS), (size_t)PtShape<HD>::SMEM, stream, mq, mk, mv, bt, max_blocks, q_start, ctx_len, tile_seq, tile_q0, num_tiles,
                                                                     (__nv_bfloat16*)out, out_stride, nq, nkv, page_size, window,
                                                                     scale * 1.4426950408889634f, cache_rows, heads_per_cta, big_boxes, nsplit, part_o, part_ml);
    if (launch_status() != 0) return launch_status();
    if (nsplit > 1)
        launch_chain(prefill_merge_splits_kernel<HD>, dim3((unsigned)(part_rows / 8)), dim3(256), (size_t)0, stream, (const float*)part_o, (const float*)part_ml,
                     q_start, tile_seq, tile_q0, (__nv_bfloat16*)out, out_stride, nq, nsplit);
    return launch_status();
}

}  // namespace aien

using namespace aien;

// Whether aien_paged_attention_prefill_tc takes these sizes (1) or the caller must use the
// mma.sync kernel (0).
AIEN_API int aien_paged_attention_prefill_tc_supports(int hd, int page_size) {
    return ((hd == 64 || hd == 128) && page_size >= 8 && page_size <= 128 && (page_size & 7) == 0 && 128 % page_size == 0) ? 1 : 0;
}

// q [q_rows, nq*hd] (leading dimension q_stride), k_cache/v_cache [cache_rows, nkv*hd] contiguous;
// the other arguments as aien_paged_attention_prefill.
// scratch (may be null), scratch_bytes: room for the partial results of key ranges, num_tiles * 128 * nq *
// splits * (hd + 2) floats; max_ctx: an upper bound of the contexts in ctx_len, known to the host;
// force_splits: 0 lets the launch choose, n > 0 asks for n ranges (refused if the scratch is too small).
AIEN_API int aien_paged_attention_prefill_tc_split(
    const void* q, long q_stride, int q_rows, const void* k_cache, const void* v_cache, int cache_rows, const int* block_table,
    int max_blocks, const int* q_start, const int* ctx_len, const int* tile_seq, const int* tile_q0, int num_tiles, void* out,
    long out_stride, int nq, int nkv, int hd, int page_size, int window, float scale, void* scratch, long scratch_bytes, int max_ctx,
    int force_splits, cudaStream_t stream) {
    if (num_tiles <= 0) return 0;
    if (!aien_paged_attention_prefill_tc_supports(hd, page_size) || nkv <= 0 || nq % nkv != 0 || q_rows <= 0 || cache_rows <= 0)
        return AIEN_E_SHAPE;
    if ((q_stride & 7) || (out_stride & 7) || ((uintptr_t)q & 15) || ((uintptr_t)k_cache & 15) || ((uintptr_t)v_cache & 15) ||
        ((uintptr_t)out & 15) || ((uintptr_t)scratch & 15))
        return AIEN_E_ALIGN;
    if (force_splits < 0 || force_splits > PT_MAX_SPLITS) return AIEN_E_SHAPE;
    CUtensorMap mq;
    static PtMaps mk, mv;                      // large: kept out of the stack; filled for every launch
    static std::mutex mu;
    std::lock_guard<std::mutex> lock(mu);
    const uint64_t kv_cols = (uint64_t)nkv * hd;
    if (!make_map(&mq, q, (uint64_t)q_rows, (uint64_t)nq * hd, (uint64_t)q_stride, 64, PT_BM)) return AIEN_E_STATE;
    for (int lv = 0; lv < 5; ++lv) {
        const uint32_t rows = (uint32_t)page_size << lv;
        if (rows > (uint32_t)PT_BN) { mk.m[lv] = mk.m[0]; mv.m[lv] = mv.m[0]; continue; }
        if (!make_map(&mk.m[lv], k_cache, (uint64_t)cache_rows, kv_cols, kv_cols, 64, rows) ||
            !make_map(&mv.m[lv], v_cache, (uint64_t)cache_rows, kv_cols, kv_cols, 64, rows))
            return AIEN_E_STATE;
    }
    // one copy for a whole block of 128 keys, when the pool has that many rows at all
    const int big_boxes = cache_rows >= PT_BN &&
                          make_map_chunked(&mk.blk, k_cache, (uint64_t)cache_rows, kv_cols, kv_cols, PT_BN, (uint32_t)(hd / 64)) &&
                          make_map_chunked(&mv.blk, v_cache, (uint64_t)cache_rows, kv_cols, kv_cols, PT_BN, (uint32_t)(hd / 64)) ? 1 : 0;
    if (!big_boxes) { mk.blk = mk.m[0]; mv.blk = mv.m[0]; }
    if (hd == 64)
        return launch_prefill_tc<64>(mq, mk, mv, big_boxes, block_table, max_blocks, q_start, ctx_len, tile_seq, tile_q0, num_tiles, out, out_stride,
                                     nq, nkv, page_size, window, scale, cache_rows, scratch, scratch_bytes, max_ctx, force_splits, stream);
    return launch_prefill_tc<128>(mq, mk, mv, big_boxes, block_table, max_blocks, q_start, ctx_len, tile_seq, tile_q0, num_tiles, out, out_stride,
                                  nq, nkv, page_size, window, scale, cache_rows, scratch, scratch_bytes, max_ctx, force_splits, stream);
}

// The same without scratch: every tile's keys in one range.
AIEN_API int aien_paged_attention_prefill_tc(
    const void* q, long q_stride, int q_rows, const void* k_cache, const void* v_cache, int cache_rows, const int* block_table,
    int max_blocks, const int* q_start, const int* ctx_len, const int* tile_seq, const int* tile_q0, int num_tiles, void* out,
    long out_stride, int nq, int nkv, int hd, int page_size, int window, float scale, cudaStream_t stream) {
    return aien_paged_attention_prefill_tc_split(q, q_stride, q_rows, k_cache, v_cache, cache_rows, block_table, max_blocks, q_start, ctx_len,
                                                 tile_seq, tile_q0, num_tiles, out, out_stride, nq, nkv, hd, page_size, window, scale,
                                                 nullptr, 0, 0, 0, stream);
}

// Reads and clears the code a bounded wait may have left (0: none; 1 producer, 2 K/V block,
// 3 query tile, 4/5 probabilities of head A/B, 6 scores, 7 block product).
AIEN_API int aien_attention_prefill_tc_error(void) {
    int v = 0, zero = 0;
    if (cudaMemcpyFromSymbol(&v, g_wait_error, sizeof(int)) != cudaSuccess) return -1;
    if (v != 0) cudaMemcpyToSymbol(g_wait_error, &zero, sizeof(int));
    return v;
}

AIEN_DEFINE_WAIT_ERROR_ADDRESS(aien_attention_prefill_tc_error_address)
