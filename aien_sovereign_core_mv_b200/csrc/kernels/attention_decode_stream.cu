// Decode attention over the paged bfloat16 cache, streamed: the same split of the keys into chunks
// of 128 absolute positions, the same arithmetic per chunk and the same merge as the kernel in
// attention_decode.cu (so the two give the same bits), but organised for bandwidth.
//
// A fixed number of CTAs (two per SM) each take segments (token, kv head, a run of consecutive
// chunks) in a strided order and stream them through a ring of three shared-memory slots:
//   warp 8      producer: for every chunk, one TMA copy per page and 64-column half of K, then of
//               V, through the block table (absent pages are fetched at an out-of-range coordinate,
//               which fills zeros), and a bulk copy of the kv head's query rows; it runs up to three
//               slots ahead of the math, across chunk and segment borders
//   warps 0-7   the math of a chunk in three phases as before: scores on mma.sync with the keys as
//               rows (each warp 16 keys), softmax per head over the chunk, V^T . P with V^T
//               fragments from transposing ldmatrix reads; the chunk's partial result goes to scratch
// K and V tiles lie as TMA writes them (rows of 128 bytes, 128-byte swizzle): the score phase
// assigns fragment rows to keys so that the two rows a quarter-warp reads differ in swizzle group.
// At the end of a segment the CTA adds the segment's chunk count to the (token, kv head) ticket;
// the CTA that completes the count merges all chunks in chunk order.  The math warps wait for the
// ticket while the producer keeps streaming.  When the launch allows 128 chunks a token or more, no
// tickets are taken and a second, small kernel behind this one merges every (token, query head) with
// many CTAs (the same sums in the same order).
//
// Needs head size 64 or 128, pages of 8..128 tokens that divide 128, at most 16 query heads per
// kv head; other shapes take the kernel in attention_decode.cu.  The cache must hold finite values
// everywhere (whole pages are loaded; a masked key meets a zero weight).  Every wait is bounded
// and reports through aien_attention_decode_stream_error.
#include "tma.cuh"
#include "attention_decode_merge.cuh"
#include <math.h>
#include <cstdlib>

namespace aien {

constexpr int DS_CHUNK = 128, DS_MATH_WARPS = 8, DS_THREADS = (DS_MATH_WARPS + 1) * 32, DS_SLOTS = 3;

struct DsMeta {            // what the producer tells the math warps about a chunk
    int zt;                // index of the token among those the launch serves; -1: no more work
    int t;                 // row of the token in q / out / positions
    int kvh, split;        // kv head, chunk index
    int lo, hi;            // first and last key of the chunk that the token sees
    int s_lo, s_hi;        // first and last chunk of the token
    int seg_chunks;        // chunks of this segment; > 0 on the segment's last chunk, else 0
    int pad[3];
};

__device__ __forceinline__ void ds_bulk_copy(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}
__device__ __forceinline__ void ds_math_sync() { asm volatile("bar.sync 1, %0;" ::"n"(DS_MATH_WARPS * 32) : "memory"); }
__device__ __forceinline__ uint4 ds_lds16(uint32_t addr) {
    uint4 r;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w) : "r"(addr));
    return r;
}
__device__ __forceinline__ void ds_mma(float c[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// HD: head size (64 or 128); NT = ceil(G / 8) head tiles
template <int HD, int NT>
__global__ void __launch_bounds__(DS_THREADS, 2)
paged_decode_stream_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                           const __nv_bfloat16* __restrict__ q, long q_stride, const int* __restrict__ block_table, int max_blocks,
                           const int* __restrict__ seq_of_token, const int* __restrict__ positions, const int* __restrict__ token_list,
                           float* __restrict__ part_out, float* __restrict__ part_ml, int* __restrict__ counters,
                           __nv_bfloat16* __restrict__ out, long out_stride, int nq, int nkv, int page_size, int window, float scale,
                           int max_splits, int T, int segs, int cache_rows, int misc_bytes, int merge_outside) {
    constexpr int HALVES = HD / 64, HS = HD / 32, NH = NT * 8;
    constexpr uint32_t TILE = DS_CHUNK * HD * 2;                  // one K or V chunk
    extern __shared__ uint8_t ds_smem[];
    const uint32_t base = (smem_u32(ds_smem) + 1023u) & ~1023u;
    uint8_t* gen = ds_smem + (base - smem_u32(ds_smem));
    const uint32_t ring = base;
    const uint32_t q_u = ring + DS_SLOTS * TILE;                  // two query buffers of NH * HD bfloat16
    constexpr uint32_t QBUF = NH * HD * 2;
    const uint32_t meta_u = q_u + 2 * QBUF;                       // two DsMeta
    const uint32_t bars = meta_u + 2 * sizeof(DsMeta);
    const uint32_t full0 = bars, empty0 = bars + 8 * DS_SLOTS;
    const uint32_t misc_u = (empty0 + 8 * DS_SLOTS + 15u) & ~15u;
    DsMeta* meta = reinterpret_cast<DsMeta*>(gen + (meta_u - base));
    float* misc = reinterpret_cast<float*>(gen + (misc_u - base));
    __shared__ int s_is_last;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int G = nq / nkv;
    const long total = (long)segs * T * nkv;      // segs: segments per (token, kv head)

    griddep_launch();
    if (tid == 0) {
        for (int i = 0; i < DS_SLOTS; ++i) { mbar_init(full0 + 8 * i, 1); mbar_init(empty0 + 8 * i, DS_MATH_WARPS); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();

    if (warp == DS_MATH_WARPS) {
        // ------------------------------------------------------------------ producer
        const int pages_per_chunk = DS_CHUNK / page_size;
        int item = 0, kc = 0;                                     // ring items issued, K items issued
        // The kernel ahead in the step writes the query rows and, in the caches, the row of each
        // token's own position; everything else this kernel reads (positions, block tables, keys of
        // earlier positions) was complete before the step's first kernel began.  So the producer
        // fills the ring with chunks that end before the token's position while the kernel ahead is
        // still running, and waits for it only before the first chunk that holds the position, or when
        // the ring is full; the query copies of the items issued by then follow the wait.  No thread
        // writes global memory before a query has arrived.
        bool waited = false;
        int npend = 0;
        const __nv_bfloat16* pend_src0 = nullptr; const __nv_bfloat16* pend_src1 = nullptr;
        uint32_t pend_dst0 = 0, pend_dst1 = 0, pend_bar0 = 0, pend_bar1 = 0;
        auto sync_ahead = [&]() {
            if (waited) return;
            griddep_wait();
            waited = true;
            if (lane == 0) {
                if (npend > 0) ds_bulk_copy(pend_dst0, pend_src0, (uint32_t)(G * HD * 2), pend_bar0);
                if (npend > 1) ds_bulk_copy(pend_dst1, pend_src1, (uint32_t)(G * HD * 2), pend_bar1);
            }
            npend = 0;
        };
        auto acquire = [&](int it) {
            if (it >= DS_SLOTS) {
                sync_ahead();                                     // the math warps cannot free a slot without a query
                mbar_wait(empty0 + 8 * (it % DS_SLOTS), ((it / DS_SLOTS) - 1) & 1, 1);
            }
        };
        // one run: chunks [s_lo + rel_begin, s_lo + rel_begin + count) of (token zt, kv head kvh)
        auto emit_run = [&](int zt, int kvh, int rel_begin, int count) {
            const int t = token_list ? token_list[zt] : zt;
            const int pos = positions[t];
            const int first = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
            const int s_lo = first / DS_CHUNK, s_hi = pos / DS_CHUNK;
            const int c_begin = s_lo + rel_begin, c_end = min(s_hi, c_begin + count - 1);
            if (c_begin > c_end) return;
            const int* bt = block_table + (size_t)(seq_of_token ? seq_of_token[t] : t) * max_blocks;
            for (int c = c_begin; c <= c_end; ++c) {
                const int chunk_base = c * DS_CHUNK;
                int row = cache_rows;                              // out of range: zeros
                if (lane < pages_per_chunk) {
                    const int key0 = chunk_base + lane * page_size, blk = key0 / page_size;
                    if (key0 <= pos && key0 + page_size > first && blk < max_blocks) {
                        const int page = bt[blk];
                        if (page >= 0) row = page * page_size;
                    }
                }
                // K item: meta, the query rows, the K pages
                if (c == s_hi || npend == 2) sync_ahead();
                acquire(item);
                const int slot_k = item % DS_SLOTS;
                if (lane == 0) {
                    DsMeta m;
                    m.zt = zt; m.t = t; m.kvh = kvh; m.split = c;
                    m.lo = max(first, chunk_base); m.hi = min(pos, chunk_base + DS_CHUNK - 1);
                    m.s_lo = s_lo; m.s_hi = s_hi;
                    m.seg_chunks = (c == c_end) ? (c_end - c_begin + 1) : 0;
                    meta[kc & 1] = m;
                    mbar_expect_tx(full0 + 8 * slot_k, TILE + (uint32_t)(G * HD * 2));
                    const __nv_bfloat16* q_src = q + (size_t)t * q_stride + (size_t)kvh * G * HD;
                    if (waited) ds_bulk_copy(q_u + (kc & 1) * QBUF, q_src, (uint32_t)(G * HD * 2), full0 + 8 * slot_k);
                    else if (npend == 0) { pend_src0 = q_src; pend_dst0 = q_u + (kc & 1) * QBUF; pend_bar0 = full0 + 8 * slot_k; }
                    else { pend_src1 = q_src; pend_dst1 = q_u + (kc & 1) * QBUF; pend_bar1 = full0 + 8 * slot_k; }
                }
                if (!waited) ++npend;
                __syncwarp();
                if (lane < pages_per_chunk)
                    for (int h = 0; h < HALVES; ++h)
                        tma_load_2d(ring + slot_k * TILE + h * (DS_CHUNK * 128) + lane * page_size * 128, &map_k, full0 + 8 * slot_k,
                                    kvh * HD + h * 64, row);
                ++item; ++kc;
                // V item
                acquire(item);
                const int slot_v = item % DS_SLOTS;
                if (lane == 0) mbar_expect_tx(full0 + 8 * slot_v, TILE);
                __syncwarp();
                if (lane < pages_per_chunk)
                    for (int h = 0; h < HALVES; ++h)
                        tma_load_2d(ring + slot_v * TILE + h * (DS_CHUNK * 128) + lane * page_size * 128, &map_v, full0 + 8 * slot_v,
                                    kvh * HD + h * 64, row);
                ++item;
            }
        };
        if (segs > 0) {
            for (long w = blockIdx.x; w < total; w += gridDim.x) {
                // w = (seg * T + zt) * nkv + kvh: neighbours in the order share a token
                const int kvh = (int)(w % nkv);
                const long r1 = w / nkv;
                const int zt = (int)(r1 % T), seg = (int)(r1 / T);
                const int t = token_list ? token_list[zt] : zt;
                const int pos = positions[t];
                const int first = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
                // the token's own chunks are cut into `segs` runs of equal length (the last ones may be empty)
                const int per_seg = (pos / DS_CHUNK - first / DS_CHUNK + segs) / segs;
                emit_run(zt, kvh, seg * per_seg, per_seg);
            }
        } else {
            // More (token, kv head) pairs than CTAs (T <= 256): the chunks of all pairs, in pair order,
            // are cut into gridDim.x equal ranges, so a CTA takes the tail of one pair, whole pairs and
            // the head of another, and contexts of different lengths weigh what they hold.  Lane l keeps
            // the chunk counts of tokens l, l + 32, ... and how many chunks lie before each.
            int nch[8], pre[8], all = 0;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const int zt = j * 32 + lane;
                int n = 0;
                if (zt < T) {
                    const int pos = positions[token_list ? token_list[zt] : zt];
                    const int first = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
                    n = pos / DS_CHUNK - first / DS_CHUNK + 1;
                }
                int incl = n;
#pragma unroll
                for (int o = 1; o < 32; o <<= 1) {
                    const int up = __shfl_up_sync(0xffffffffu, incl, o);
                    if (lane >= o) incl += up;
                }
                nch[j] = n; pre[j] = all + incl - n;
                all += __shfl_sync(0xffffffffu, incl, 31);
            }
            const long chunks = (long)all * nkv;
            long at = chunks * blockIdx.x / gridDim.x;
            const long end = chunks * (blockIdx.x + 1) / gridDim.x;
            while (at < end) {
                int zt = -1, before = 0, n = 0;
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const bool mine = nch[j] > 0 && (long)nkv * pre[j] <= at && at < (long)nkv * (pre[j] + nch[j]);
                    const unsigned m = __ballot_sync(0xffffffffu, mine);
                    if (m != 0u) {
                        const int src = __ffs(m) - 1;
                        zt = j * 32 + src;
                        before = __shfl_sync(0xffffffffu, pre[j], src);
                        n = __shfl_sync(0xffffffffu, nch[j], src);
                    }
                }
                if (zt < 0) break;                                 // cannot happen: every chunk index belongs to a token
                const int rem = (int)(at - (long)nkv * before);
                const int kvh = rem / n, rel = rem - kvh * n;
                const int count = (int)min((long)(n - rel), end - at);
                emit_run(zt, kvh, rel, count);
                at += count;
            }
        }
        sync_ahead();
        // the end mark travels like a K item
        acquire(item);
        if (lane == 0) {
            DsMeta m = {};
            m.zt = -1;
            meta[kc & 1] = m;
            mbar_arrive(full0 + 8 * (item % DS_SLOTS));
        }
        return;
    }

    // ---------------------------------------------------------------------- math warps
    const int g = lane >> 2, c4 = lane & 3;
    // Row strides padded so that neither the writers nor the readers of a phase meet in a bank.
    constexpr int SC_LD = DS_CHUNK + 4, PT_LD = DS_CHUNK + 8;
    float* Sc = misc;                                              // scores [NH][SC_LD]
    float* Hm = Sc + NH * SC_LD;                                   // per head max, then denominator
    float* Hl = Hm + NH;
    __nv_bfloat16* Pt = reinterpret_cast<__nv_bfloat16*>(Hl + NH);   // probabilities [NH][PT_LD]
    int item = 0;
    for (int kc = 0;; ++kc) {
        const int slot_k = item % DS_SLOTS;
        mbar_wait(full0 + 8 * slot_k, (item / DS_SLOTS) & 1, 2);
        const DsMeta m = meta[kc & 1];
        if (m.zt < 0) break;
        const uint32_t K_u = ring + slot_k * TILE;
        const int chunk_base = m.split * DS_CHUNK;

        // ---- phase 1: scores of this warp's 16 keys for every head.  Fragment row g is key
        // rho(g) = (g >> 1) | ((g & 1) << 2) of the warp's first eight, row g + 8 the same of the second eight.
        {
            const __nv_bfloat16* Qs = reinterpret_cast<const __nv_bfloat16*>(gen + (q_u + (kc & 1) * QBUF - base));
            uint4 qf[NT][HS];
#pragma unroll
            for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                for (int ds = 0; ds < HS; ++ds) {
                    const int h = nt * 8 + g;
                    qf[nt][ds] = h < G ? *reinterpret_cast<const uint4*>(Qs + h * HD + ds * 32 + c4 * 8) : make_uint4(0u, 0u, 0u, 0u);
                }
            const int rho = (g >> 1) | ((g & 1) << 2);
            const int r0 = warp * 16 + rho, r1 = r0 + 8;
            const int kj0 = chunk_base + r0, kj1 = chunk_base + r1;
            const bool ok0 = kj0 >= m.lo && kj0 <= m.hi, ok1 = kj1 >= m.lo && kj1 <= m.hi;
            float S[NT][4];
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) S[nt][0] = S[nt][1] = S[nt][2] = S[nt][3] = 0.f;
#pragma unroll
            for (int ds = 0; ds < HS; ++ds) {
                const uint32_t off = (uint32_t)(ds >> 1) * (DS_CHUNK * 128) + (uint32_t)(((((ds & 1) << 2) + c4) ^ (rho & 7)) << 4);
                const uint4 ka = ds_lds16(K_u + r0 * 128 + off), kb = ds_lds16(K_u + r1 * 128 + off);
#pragma unroll
                for (int nt = 0; nt < NT; ++nt) {
                    ds_mma(S[nt], ka.x, kb.x, ka.y, kb.y, qf[nt][ds].x, qf[nt][ds].y);
                    ds_mma(S[nt], ka.z, kb.z, ka.w, kb.w, qf[nt][ds].z, qf[nt][ds].w);
                }
            }
            // S[nt][e]: key r0, head nt*8+2c+e;  S[nt][2+e]: key r1, same head
#pragma unroll
            for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const int h = nt * 8 + 2 * c4 + e;
                    Sc[h * SC_LD + r0] = ok0 ? S[nt][e] * scale : -INFINITY;
                    Sc[h * SC_LD + r1] = ok1 ? S[nt][2 + e] * scale : -INFINITY;
                }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(empty0 + 8 * slot_k);           // K and the query buffer may be refilled
        ++item;
        ds_math_sync();
        // ---- phase 2: per head, maximum, probabilities and denominator over the chunk (keys in order)
        for (int h = warp; h < NH; h += DS_MATH_WARPS) {
            float sv[DS_CHUNK / 32];
            float mx = -INFINITY;
#pragma unroll
            for (int i = 0; i < DS_CHUNK / 32; ++i) { sv[i] = Sc[h * SC_LD + i * 32 + lane]; mx = fmaxf(mx, sv[i]); }
            mx = warp_max(mx);
            float sum = 0.f;
#pragma unroll
            for (int i = 0; i < DS_CHUNK / 32; ++i) {
                const float pv = (mx == -INFINITY || sv[i] == -INFINITY) ? 0.f : expf(sv[i] - mx);
                sum += pv;
                Pt[h * PT_LD + i * 32 + lane] = __float2bfloat16_rn(pv);
            }
            sum = warp_sum(sum);
            if (lane == 0) { Hm[h] = mx; Hl[h] = sum; }
        }
        const int slot_v = item % DS_SLOTS;
        mbar_wait(full0 + 8 * slot_v, (item / DS_SLOTS) & 1, 3);
        ds_math_sync();                                            // P is visible
        // ---- phase 3: out^T[dims, heads] = V^T[dims, keys] . P[keys, heads]; a warp owns 16 dims at a time
        const uint32_t V_u = ring + slot_v * TILE;
        for (int mt = warp; mt * 16 < HD; mt += DS_MATH_WARPS) {
            float oacc[NT][4];
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) oacc[nt][0] = oacc[nt][1] = oacc[nt][2] = oacc[nt][3] = 0.f;
            // this lane's row address for ldmatrix: key (lane&7) + 8*(lane>>4) of each 16, 16-byte piece 2*mt + ((lane>>3)&1)
            const int krow = (lane & 7) + ((lane >> 4) << 3);
            const int piece = mt * 2 + ((lane >> 3) & 1);
            const uint32_t vbase = V_u + (uint32_t)(piece >> 3) * (DS_CHUNK * 128) + krow * 128 + (uint32_t)(((piece & 7) ^ (krow & 7)) << 4);
#pragma unroll
            for (int ks = 0; ks < DS_CHUNK / 16; ++ks) {
                uint32_t a0, a1, a2, a3;
                asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                             : "=r"(a0), "=r"(a1), "=r"(a2), "=r"(a3) : "r"(vbase + ks * 16 * 128));
#pragma unroll
                for (int nt = 0; nt < NT; ++nt) {
                    const uint32_t* prow = reinterpret_cast<const uint32_t*>(Pt + (nt * 8 + g) * PT_LD + ks * 16);
                    ds_mma(oacc[nt], a0, a1, a2, a3, prow[c4], prow[c4 + 4]);
                }
            }
#pragma unroll
            for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const int h = nt * 8 + 2 * c4 + e;
                    if (h < G) {
                        const size_t row = ((size_t)m.zt * nq + m.kvh * G + h) * max_splits + m.split;
                        part_out[row * HD + mt * 16 + g] = oacc[nt][e];
                        part_out[row * HD + mt * 16 + g + 8] = oacc[nt][2 + e];
                    }
                }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(empty0 + 8 * slot_v);
        ++item;
        if (tid < G) {
            const size_t row = ((size_t)m.zt * nq + m.kvh * G + tid) * max_splits + m.split;
            part_ml[row * 2] = Hm[tid];
            part_ml[row * 2 + 1] = Hl[tid];
        }
        if (m.seg_chunks > 0 && !merge_outside) {
            // ---- the segment is done: ticket; the CTA that completes the count merges the chunks
            ds_math_sync();                                        // every thread's partial results are written
            const bool solo = m.seg_chunks == m.s_hi - m.s_lo + 1; // this CTA made every chunk of the token: no ticket
            if (!solo) {
                if (tid == 0) {
                    __threadfence();                               // ... and ordered before the ticket, device-wide
                    const int before = atomicAdd(&counters[(size_t)m.zt * nkv + m.kvh], m.seg_chunks);
                    s_is_last = before + m.seg_chunks == m.s_hi - m.s_lo + 1;
                    if (s_is_last) counters[(size_t)m.zt * nkv + m.kvh] = 0;     // ready for the next launch
                }
                ds_math_sync();
            }
            if (solo || s_is_last) {
                if (!solo) __threadfence();
                ad_merge_chunks<NH, 1>(misc, part_out, part_ml, out + (size_t)m.t * out_stride + (size_t)m.kvh * G * HD,
                                    (size_t)m.zt * nq + m.kvh * G, G, HD, max_splits, m.s_lo, m.s_hi - m.s_lo + 1, tid,
                                    DS_MATH_WARPS * 32, [] { ds_math_sync(); });
            }
            ds_math_sync();                                        // the scratch is free for the next chunk
        }
    }
}

// Shared memory of one CTA: alignment slack, the ring, two query buffers, two DsMeta, the barriers,
// and the scratch of the phases or of the merge, whichever is larger.  Up to 113 KB two CTAs share an SM.
constexpr size_t DS_SMEM_LIMIT = 200 * 1024;
// From how many chunks per token on (the launch's limit, not the token's own count) the merge is a kernel of its
// own behind this one (paged_decode_merge_kernel) and this kernel takes no tickets.  Measured on the 32q/8kv x 128
// shape, merge inside -> outside: one request of 32,768 keys 41.8 -> 28.1 us, of 16,384 keys 17.8 -> 14.2 us, four of
// 32,768 109.4 -> 93.1 us, eight of 16,384 98.4 -> 94.5 us; at 64 chunks (sixteen of 8,192) 93.7 -> 97.5 us, so from 128.
// AIEN_B200_DECODE_MERGE_KERNEL_FROM overrides the limit.
constexpr int DS_MERGE_OUTSIDE_FROM = 128;
static bool ds_merge_outside(int max_splits) {
    static int from = -1;
    if (from < 0) { const char* e = getenv("AIEN_B200_DECODE_MERGE_KERNEL_FROM"); from = (e && atoi(e) > 0) ? atoi(e) : DS_MERGE_OUTSIDE_FROM; }
    return max_splits >= from && ad_merge_kernel_smem(max_splits) <= 48 * 1024;
}
static size_t ds_smem_bytes(int hd, int nt, int G, int max_splits, size_t* misc_out) {
    const size_t NH = (size_t)nt * 8;
    const size_t loop_bytes = ((size_t)(DS_CHUNK + 4) * NH + 2 * NH) * 4 + NH * (DS_CHUNK + 8) * 2;
    const size_t merge_bytes = ds_merge_outside(max_splits) ? 0 : ad_merge_scratch_floats(max_splits, G, hd) * 4;
    const size_t misc_bytes = ((loop_bytes > merge_bytes ? loop_bytes : merge_bytes) + 127) & ~(size_t)127;
    if (misc_out) *misc_out = misc_bytes;
    return 1024 + (size_t)DS_SLOTS * DS_CHUNK * hd * 2 + 2 * NH * hd * 2 + 2 * sizeof(DsMeta) + 16 * DS_SLOTS + 16 + misc_bytes;
}

static int ds_num_sms() {
    static int n = 0;
    if (n == 0) {
        int dev = 0;
        if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    }
    return n;
}

// Into how many segments the chunks of one (token, kv head) pair are cut, from the launch's shape
// alone: as many as still give every CTA at most one segment; one (the whole token, which then
// needs no ticket) when there are more pairs than CTAs.  The kernel cuts each token's own chunk
// count into that many equal runs.  Measured on the 32q/8kv x 128 shape at 1,030 keys (9 chunks),
// batches 4 / 8 / 16 / 32 / 64 are best or within 1 % of best at 1 / 3 / 5 / 9 / 9 chunks per
// segment, and 16 requests of 8,192 keys at 32: what this rule gives.
static int ds_segments_per_pair(long pairs, int max_splits, long slots) {
    if (pairs >= slots) return 1;
    const long segs = slots / pairs;
    return (int)(segs < max_splits ? segs : max_splits);
}

template <int HD, int NT>
static int launch_decode_stream(const CUtensorMap& mk, const CUtensorMap& mv, const void* q, long q_stride, const int* bt, int max_blocks,
                                const int* seq_of_token, const int* positions, const int* token_list, float* part_out, float* part_ml,
                                int* counters, void* out, long out_stride, int nq, int nkv, int page_size, int window, float scale,
                                int max_splits, int T, int cache_rows, cudaStream_t stream) {
    size_t misc_bytes = 0;
    const size_t smem = ds_smem_bytes(HD, NT, nq / nkv, max_splits, &misc_bytes);
    if (smem > DS_SMEM_LIMIT) return AIEN_E_SHAPE;
    auto kern = paged_decode_stream_kernel<HD, NT>;
    static size_t configured = 0;
    if (smem > configured) {
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) return AIEN_E_STATE;
        configured = smem;
    }
    const long slots = 2L * ds_num_sms();
    const bool outside = ds_merge_outside(max_splits);
    int segs = ds_segments_per_pair((long)T * nkv, max_splits, slots);
    if (const char* e = getenv("AIEN_B200_DECODE_SEGMENTS")) { const int v = atoi(e); if (v > 0 && v <= max_splits) segs = v; }
    // more pairs than CTAs: equal ranges of chunks instead of whole pairs (segs = 0 tells the kernel); AIEN_B200_DECODE_BALANCED=0: off
    static int balanced = -1;
    if (balanced < 0) { const char* e = getenv("AIEN_B200_DECODE_BALANCED"); balanced = (e && e[0] == '0') ? 0 : 1; }
    // (measured, 32q/8kv x 128 at 1,030 keys, whole pairs -> ranges, the kernel alone: batch 48 the same, 64 54.3 -> 53.5 us,
    // 96 81.2 -> 76.9 us, 128 108.0 -> 99.0 us; inside a decode step of 36 layers: batch 48 5.26 -> 5.03 ms, 64 5.69 -> 5.73 ms,
    // 96 7.09 -> 7.02 ms, 128 8.37 -> 8.25 ms.  A range shares pairs with its neighbours, and every shared pair is a ticket
    // and a merge more: so only when whole pairs would leave a fifth of the CTA rounds empty, or take three rounds or more.)
    const long pairs = (long)T * nkv, rounds = (pairs + slots - 1) / slots;
    if (balanced && segs == 1 && pairs > slots && (pairs * 10 < slots * rounds * 8 || rounds >= 3) && T <= 256 &&
        getenv("AIEN_B200_DECODE_SEGMENTS") == nullptr) segs = 0;
    const long total = segs > 0 ? (long)segs * T * nkv : slots;
    const unsigned grid = (unsigned)(total < slots ? total : slots);
    launch_chain(kern, dim3(grid), dim3(DS_THREADS), smem, stream, mk, mv, (const __nv_bfloat16*)q, q_stride, bt, max_blocks, seq_of_token,
                 positions, token_list, part_out, part_ml, counters, (__nv_bfloat16*)out, out_stride, nq, nkv, page_size, window, scale,
                 max_splits, T, segs, cache_rows, (int)misc_bytes, outside ? 1 : 0);
    if (outside)
        launch_decode_merge<HD>(part_out, part_ml, positions, token_list, (__nv_bfloat16*)out, out_stride, nq, window, max_splits,
                                DS_CHUNK, T, stream);
    return launch_status();
}

}  // namespace aien

using namespace aien;

// Whether aien_paged_attention_decode_stream takes these sizes (1) or the caller must use
// aien_paged_attention_decode (0).
AIEN_API int aien_paged_attention_decode_stream_supports(int nq, int nkv, int hd, int page_size, int max_splits) {
    if (nkv <= 0 || nq % nkv != 0 || nq / nkv > 16) return 0;
    if (!(hd == 64 || hd == 128) || page_size < 8 || page_size > 128 || (page_size & 7) || 128 % page_size != 0) return 0;
    return (max_splits > 0 && ds_smem_bytes(hd, (nq / nkv + 7) / 8, nq / nkv, max_splits, nullptr) <= DS_SMEM_LIMIT) ? 1 : 0;
}

// Arguments as aien_paged_attention_decode, plus the number of rows of the caches ([cache_rows, nkv*hd]).
AIEN_API int aien_paged_attention_decode_stream(
    const void* q, long q_stride, const void* k_cache, const void* v_cache, int cache_rows, const int* block_table, int max_blocks,
    const int* seq_of_token, const int* positions, const int* token_list, void* out, long out_stride, float* part_out,
    float* part_ml, int* counters, int nq, int nkv, int hd, int page_size, int window, float scale, int max_splits, int T,
    cudaStream_t stream) {
    if (T <= 0) return 0;
    if (max_splits <= 0 || cache_rows <= 0 || !aien_paged_attention_decode_stream_supports(nq, nkv, hd, page_size, max_splits)) return AIEN_E_SHAPE;
    if ((q_stride & 7) || ((uintptr_t)q & 15) || ((uintptr_t)k_cache & 15) || ((uintptr_t)v_cache & 15)) return AIEN_E_ALIGN;
    CUtensorMap mk, mv;
    const uint64_t kv_cols = (uint64_t)nkv * hd;
    if (!make_map(&mk, k_cache, (uint64_t)cache_rows, kv_cols, kv_cols, 64, (uint32_t)page_size) ||
        !make_map(&mv, v_cache, (uint64_t)cache_rows, kv_cols, kv_cols, 64, (uint32_t)page_size))
        return AIEN_E_STATE;
    const int NT = (nq / nkv + 7) / 8;
#define DS_CASE(HDV, NTV)                                                                                                  \
    if (hd == HDV && NT == NTV)                                                                                            \
        return launch_decode_stream<HDV, NTV>(mk, mv, q, q_stride, block_table, max_blocks, seq_of_token, positions,        \
                                              token_list, part_out, part_ml, counters, out, out_stride, nq, nkv, page_size, \
                                              window, scale, max_splits, T, cache_rows, stream);
    DS_CASE(64, 1) DS_CASE(64, 2) DS_CASE(128, 1) DS_CASE(128, 2)
#undef DS_CASE
    return AIEN_E_SHAPE;
}

// Reads and clears the code a bounded wait may have left (0: none; 1 producer, 2 K tile, 3 V tile).
AIEN_API int aien_attention_decode_stream_error(void) {
    int v = 0, zero = 0;
    if (cudaMemcpyFromSymbol(&v, g_wait_error, sizeof(int)) != cudaSuccess) return -1;
    if (v != 0) cudaMemcpyToSymbol(g_wait_error, &zero, sizeof(int));
    return v;
}

AIEN_DEFINE_WAIT_ERROR_ADDRESS(aien_attention_decode_stream_error_address)
