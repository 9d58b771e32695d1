// Paged causal attention for prompt portions on the 5th-generation tensor cores (tcgen05).
//
// A CTA owns 128 query tokens of one request and one query head (the 128 lanes of tensor memory)
// and walks the request's keys in tiles of 128 tokens, fetched page by page from the cache by TMA
// through the block table: one copy per page for K and one for V, whatever the page size, through
// tensor maps of rank 5 and 4 that view the cache so that a page lands in the order the MMA
// descriptors can walk (K: [8 tokens][64-column block][8 x 128 bytes], the groups of 8 keys of a block
// at one stride over the whole tile; V: [page][block][token][128 bytes], each MMA taking 16 keys of
// one page).  Per tile:
//
//     S  = Q K^T           tcgen05.mma, Q and K both K-major in shared memory, S in TMEM
//     P  = 2^(S c - m)     softmax warps: two threads per query row read its half row of S from TMEM
//                          once (no shuffles), float32 statistics, P rounded to bfloat16 and written
//                          back to TMEM over the first quarter of S (tcgen05.st, two keys per column)
//     O += P V             tcgen05.mma with its A operand (P) in TMEM, V as it lies in the cache (head
//                          dimension contiguous = MN-major B operand), O accumulated in TMEM over all
//                          tiles.  P never passes through shared memory, whose bandwidth bounds the kernel.
//
// m is the maximum the row's exponentials are taken against.  It follows the row's true maximum
// lazily: only when a tile exceeds it by more than 2^8 is it moved and the accumulated O (in TMEM)
// and the row sum rescaled, which after the first tiles of a row hardly ever happens; the result
// is the same sum, since numerator and denominator carry the same factor.
//
// The tiles alternate between two sets of softmax warps, each with its own S/P buffer and O
// accumulator in TMEM (2 x 128 + 2 x HD columns) and row statistics: two independent online
// softmaxes over the even and the odd tiles, merged at the end like the parts of a cut row.  One
// set's exponentials (the MUFU pipe) run beside the other's passes over S, the MMAs of both and the
// loads of later tiles.  K and V tiles share one ring of shared-memory slots, filled in the order the
// MMA warp takes them (K_0, K_1, then V_j and K_{j+2}: S of tile j+2 follows PV of tile j into the
// buffer that held S and P of tile j).  Warps (576 threads): 0 TMA producer, 1 MMA issuer and TMEM
// owner, 2..9 and 10..17 the softmax sets (warp w owns TMEM lanes 32 (w % 4) .. +31; two warps of a
// set share a lane quarter and split the columns).
//
// Reference: clockwork/kernels/attention.py:68-96 (gather the context through one block table, then
// dense causal attention with the query aligned to the end of the context, :45-65) and
// clockwork/engine/model.py:103-118.  One launch covers every portion of the batch: the host lists
// (request, first query row) work items, one per 128 query tokens; a decoded token is a portion of
// length one and may ride along.
//
// Key slots past the end of a request's context are fetched from page 0 and multiplied by
// probabilities that are exactly zero; the cache pool is zero-initialised and only ever holds
// finite values, so they cannot leak.  Every wait is bounded (CW_ST_WAIT_TIMEOUT in the status
// words, then the kernel frees TMEM and returns).
#include <type_traits>
#include "tc_common.cuh"

#define AQ 128  // query rows per CTA
#define AK 128  // keys per tile
#define A_THREADS 576  // TMA producer, MMA issuer, two sets of 8 softmax warps
#define A_MAX_SMEM (227 * 1024)
#define PREFILL_MAX_PARTS 8  // parts that a long row of keys may be cut into
#define LAZY_STEP 8.0f  // log2 of how far a tile's maximum may exceed the one in use before the row is rescaled

struct PrefillTcParams {
    bf16* out;
    const int* block_tables; const int* q_start; const int* ctx_lens;
    const int* item_seq; const int* item_q0;
    // Long rows of keys cut into parts (or null: none is).  item_split[i] = (first item of i's group) << 8 |
    // parts; the group's items are consecutive, item i being part i - first.  A part leaves its
    // unnormalised O and (m, l) per row in part_o / part_ml (indexed by item and head) and counts itself
    // in counters[first * nh + head] (zero between launches); the last one to arrive merges them all.
    const int* item_split; float* part_o; float* part_ml; int* counters;
    int nh, nkv, page_size, page_shift, max_blocks, num_pages;
    float scale; int window;
    int* status;
};

template <int HD>
struct ACfg {
    static constexpr int CB = HD / 64;                  // 64-element (128-byte) column blocks per row
    static constexpr int BLOCK_BYTES = 128 * 128;       // [128 rows][64 bf16], 128-byte swizzle
    static constexpr int Q_BYTES = CB * BLOCK_BYTES;
    static constexpr int SLOT_BYTES = CB * BLOCK_BYTES;  // one K or one V tile
    static constexpr int TAIL_BYTES = 256 + 2048;  // barriers, exchange of row statistics
    static constexpr int FIT = (A_MAX_SMEM - TAIL_BYTES - Q_BYTES) / SLOT_BYTES;
    static constexpr int NSLOTS = FIT > 8 ? 8 : FIT;
    static constexpr int SMEM_BYTES = Q_BYTES + NSLOTS * SLOT_BYTES + TAIL_BYTES;
    static constexpr int O_COL = 2 * AK;                 // S buffers at columns 0 and 128, the two O accumulators after them
    static constexpr int TMEM_COLS = 512;
    static_assert(NSLOTS >= 4, "too few key/value slots");
    static_assert(O_COL + 2 * HD <= TMEM_COLS, "accumulators do not fit in tensor memory");
};

__device__ __forceinline__ void tma_load_5d(uint32_t dst, const CUtensorMap* map, int x, int y, int z, int w, int v, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.5d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6, %7}], [%2];"
        ::"r"(dst), "l"(map), "r"(bar), "r"(x), "r"(y), "r"(z), "r"(w), "r"(v)
        : "memory");
}
// K-major operand, 128-byte swizzle, with the groups of 8 rows `group_bytes` apart (tc_common's form has 1024).
__device__ __forceinline__ uint64_t smem_desc_sw128_groups(uint32_t addr, uint32_t group_bytes) {
    uint64_t d = 0;
    d |= (uint64_t)((addr >> 4) & 0x3FFF);
    d |= (uint64_t)1 << 16;
    d |= (uint64_t)((group_bytes >> 4) & 0x3FFF) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}
__device__ __forceinline__ void tma_load_4d(uint32_t dst, const CUtensorMap* map, int x, int y, int z, int w, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
        ::"r"(dst), "l"(map), "r"(bar), "r"(x), "r"(y), "r"(z), "r"(w)
        : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, float* v) {
    uint32_t r[32];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
        "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}
// Descriptor of an MN-major operand with the 128-byte swizzle: rows of the K dimension are 128 bytes
// (64 contiguous elements of the MN dimension), groups of 8 rows are `group_bytes` apart (stride byte
// offset) and the next 64 elements of the MN dimension lie `mn_block_bytes` further (leading byte offset).
__device__ __forceinline__ uint64_t smem_desc_mn_sw128(uint32_t addr, uint32_t mn_block_bytes, uint32_t group_bytes) {
    uint64_t d = 0;
    d |= (uint64_t)((addr >> 4) & 0x3FFF);
    d |= (uint64_t)((mn_block_bytes >> 4) & 0x3FFF) << 16;
    d |= (uint64_t)((group_bytes >> 4) & 0x3FFF) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}
__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const float* v) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
        ::"r"(taddr), "r"(__float_as_uint(v[0])), "r"(__float_as_uint(v[1])), "r"(__float_as_uint(v[2])),
          "r"(__float_as_uint(v[3])), "r"(__float_as_uint(v[4])), "r"(__float_as_uint(v[5])), "r"(__float_as_uint(v[6])),
          "r"(__float_as_uint(v[7])), "r"(__float_as_uint(v[8])), "r"(__float_as_uint(v[9])), "r"(__float_as_uint(v[10])),
          "r"(__float_as_uint(v[11])), "r"(__float_as_uint(v[12])), "r"(__float_as_uint(v[13])), "r"(__float_as_uint(v[14])),
          "r"(__float_as_uint(v[15]))
        : "memory");
    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}
// This lane's row of an accumulator in tensor memory times alpha (rare: a rolled loop over 16 columns
// at a time, so that it takes few registers from the softmax loop around it).
template <int COLS>
__device__ __forceinline__ void rescale_o(uint32_t taddr, float alpha) {
#pragma unroll 1
    for (int c = 0; c < COLS; c += 16) {
        float v[16];
        tmem_ld16(taddr + c, v);
#pragma unroll
        for (int i = 0; i < 16; ++i) v[i] *= alpha;
        tmem_st16(taddr + c, v);
    }
}
// D (+)= A B with A in tensor memory: lane i holds row i, a 32-bit column two consecutive bfloat16 of the
// inner dimension (the lower half first), so 16 of them take 8 columns.
__device__ __forceinline__ void umma_bf16_a_tmem(uint32_t tmem_d, uint32_t tmem_a, uint64_t bdesc, uint32_t idesc,
                                                 uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
        ::"r"(tmem_d), "r"(tmem_a), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// A named barrier of n threads that also tells every one of them whether all came with `pred` true.
__device__ __forceinline__ bool bar_and(int id, int n, bool pred) {
    uint32_t all;
    asm volatile("{ .reg .pred p, q; setp.ne.u32 q, %3, 0; bar.red.and.pred p, %1, %2, q; selp.u32 %0, 1, 0, p; }"
                 : "=r"(all)
                 : "r"(id), "r"(n), "r"((uint32_t)pred)
                 : "memory");
    return all != 0;
}
__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

template <int HD>
__global__ void __launch_bounds__(A_THREADS, 1)  // (18 warps: five on one scheduler, whose 16,384 registers allow 96 per thread)
attn_prefill_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                       const __grid_constant__ CUtensorMap map_v, const PrefillTcParams p) {
    using C = ACfg<HD>;
    // the swizzled tiles need a 1024-byte aligned base; the declaration asks for it and the kernel
    // checks it instead of rounding up, because the tiles leave no kilobyte to spare
    extern __shared__ __align__(1024) uint8_t smem[];
    if (smem_u32(smem) & 1023) {
        if (threadIdx.x == 0) cw_report(p.status, CW_ST_SMEM_ALIGN, blockIdx.x, (int)(smem_u32(smem) & 1023));
        return;
    }
    uint8_t* q_s = smem;
    uint8_t* slots = q_s + C::Q_BYTES;
    uint64_t* bars = (uint64_t*)(slots + C::NSLOTS * C::SLOT_BYTES);
    // bars: q_full, -, s_full[2], o_full[2], p_full[2], -[2], full[NSLOTS], empty[NSLOTS]
    uint32_t* tmem_slot = (uint32_t*)(bars + 10 + 2 * C::NSLOTS);
    volatile int* give_up = (volatile int*)(tmem_slot + 1);
    volatile int* last_part = give_up + 1;
    float* xchg = (float*)(bars + 32);   // [2 sets][2 halves][128]: row maxima and, at the end, row sums and set 1's (m, l)

    // Work items, portion bounds, context lengths and block tables are inputs of the step, written
    // before its first kernel; only q and the newest keys and values come from the preceding kernels.
    // So everything up to the first TMA load runs while the preceding kernel finishes, and only the
    // producer warp, whose loads are the kernel's only reads of that data, waits for it.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int h = blockIdx.x, item = blockIdx.y;
    const int s = p.item_seq[item], q0 = p.item_q0[item];
    if (s < 0) return;  // an unused entry of a work list of fixed length (captured steps): nothing is set up yet
    const int kvh = h / (p.nh / p.nkv);
    const int row0 = p.q_start[s], q_len = p.q_start[s + 1] - row0;
    const int ctx = p.ctx_lens[s];
    const int pos0 = ctx - q_len + q0;           // position of the tile's first query
    const int nq = min(AQ, q_len - q0);          // query rows in this tile
    const int kv_hi = pos0 + nq;                 // keys [.., kv_hi) are visible to the last row
    const int kv_lo = p.window > 0 ? max(0, pos0 + 1 - p.window) : 0;
    int tile_lo = kv_lo / AK * AK;               // key tiles start at multiples of 128 whatever the portion
    int ntiles = (kv_hi - tile_lo + AK - 1) / AK;
    const int split_word = p.item_split != nullptr ? p.item_split[item] : (item << 8) | 1;
    const int parts = split_word & 0xFF, first_item = split_word >> 8;
    if (parts < 1 || parts > PREFILL_MAX_PARTS || first_item < 0 || first_item > item || item - first_item >= parts) {
        if (threadIdx.x == 0) cw_report(p.status, CW_ST_SPLIT_RANGE, item, split_word);
        return;
    }
    if (parts > 1) {  // this CTA's share of the tiles (it may be empty)
        const int per = (ntiles + parts - 1) / parts, begin = (item - first_item) * per;
        ntiles = max(0, min(ntiles, begin + per) - begin);
        tile_lo += begin * AK;
    }

    const uint32_t q_full = smem_u32(bars);
    const uint32_t s_full0 = smem_u32(bars + 2), o_full0 = smem_u32(bars + 4);
    const uint32_t p_full0 = smem_u32(bars + 6);
    const uint32_t full0 = smem_u32(bars + 10), empty0 = smem_u32(bars + 10 + C::NSLOTS);
    if (tid == 0) {
        mbar_init(q_full, 1);
        for (int b = 0; b < 2; ++b) {
            mbar_init(s_full0 + 8 * b, 1);
            mbar_init(o_full0 + 8 * b, 1);
            mbar_init(p_full0 + 8 * b, 256);
        }
        for (int i = 0; i < C::NSLOTS; ++i) {
            mbar_init(full0 + 8 * i, 1);
            mbar_init(empty0 + 8 * i, 1);
        }
        *give_up = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) tmem_alloc(smem_u32(tmem_slot), C::TMEM_COLS);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ---- TMA producer: Q once, then K and V tiles in the order the MMA warp takes them ------------
        // K_0, K_1, then (V_j, K_{j+2}) for every tile j: the scores run two tiles ahead of the
        // probabilities.  Lane i fetches page i of a tile: it reads the page's number from the block
        // table ahead of its use (so that the read's latency is hidden) and issues that page's copies itself.
        if (lane < 3) {
            const CUtensorMap* m = lane == 0 ? &map_q : (lane == 1 ? &map_k : &map_v);
            asm volatile("prefetch.tensormap [%0];" ::"l"(m) : "memory");
        }
        const int* table = p.block_tables + (size_t)s * p.max_blocks;
        const int pages_per_tile = AK >> p.page_shift;  // at most 16
        auto page_of = [&](int j) -> int {
            // slots past the context: any finite data will do, their probabilities are zero
            const int pos = tile_lo + j * AK + lane * p.page_size;
            const int blk = pos >> p.page_shift;
            return (j < ntiles && lane < pages_per_tile && pos < kv_hi && blk < p.max_blocks) ? table[blk] : 0;
        };
        int pg_v = page_of(0), pg_1 = page_of(1), pg_2 = page_of(2);  // this lane's page of tiles j, j+1, j+2
        asm volatile("griddepcontrol.wait;" ::: "memory");
        if (lane == 0) {
            mbar_expect_tx(q_full, C::Q_BYTES);
            for (int cb = 0; cb < C::CB; ++cb)
                tma_load_2d(smem_u32(q_s + cb * C::BLOCK_BYTES), &map_q, h * HD + cb * 64, row0 + q0, q_full);
        }
        int t = 0;
        auto load = [&](int page, bool is_v) -> bool {
            if (page < 0 || page >= p.num_pages) {
                cw_report(p.status, CW_ST_PAGE_RANGE, s, page);
                page = 0;
            }
            const int slot = t % C::NSLOTS;
            bool ok = mbar_wait(empty0 + 8 * slot, ((t / C::NSLOTS) & 1) ^ 1, give_up);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) return false;
            const uint32_t bar = full0 + 8 * slot;
            const uint32_t dst0 = smem_u32(slots + slot * C::SLOT_BYTES);
            if (lane == 0) mbar_expect_tx(bar, C::SLOT_BYTES);
            __syncwarp();
            if (lane < pages_per_tile) {
                if (is_v) {
                    // a V tile lies page by page, [page][64-column block][token][128 bytes]: one copy per page
                    tma_load_4d(dst0 + lane * C::CB * p.page_size * 128, &map_v, 0, page * p.page_size, 0, kvh, bar);
                } else {
                    // a K tile lies [8 tokens][64-column block][8 x 128 bytes]: the MMA wants the groups of 8
                    // keys of a block at one stride over all 128 keys; one copy per page here too
                    tma_load_5d(dst0 + lane * C::CB * p.page_size * 128, &map_k, 0, 0, 0, page * (p.page_size >> 3), kvh, bar);
                }
            }
            ++t;
            return true;
        };
        bool ok = true;
        if (ntiles > 0) ok = load(pg_v, false);
        if (ok && ntiles > 1) ok = load(pg_1, false);
        for (int j = 0; j < ntiles && ok; ++j) {
            const int pg_3 = page_of(j + 3);
            ok = load(pg_v, true);
            if (ok && j + 2 < ntiles) ok = load(pg_2, false);
            pg_v = pg_1;
            pg_1 = pg_2;
            pg_2 = pg_3;
        }
        if (*give_up && lane == 0) {
            // wait, bounded, for the copies still in flight before the CTA's shared memory goes away
            for (int k = max(0, t - C::NSLOTS); k < t; ++k) {
                const uint32_t bar = full0 + 8 * (k % C::NSLOTS);
                const long long t0 = clock64();
                while (!mbar_try_wait(bar, (k / C::NSLOTS) & 1) && clock64() - t0 < WAIT_CYCLES) {
                }
            }
        }
    } else if (warp == 1 && lane == 0) {
        // ---- MMA issuer --------------------------------------------------------------------------------
        constexpr uint32_t idesc_s = instr_desc(AQ, AK);
        constexpr uint32_t idesc_o = instr_desc(AQ, HD) | (1u << 16);  // B (= V) is MN-major
        bool ok = mbar_wait(q_full, 0, give_up);
        int t = 0;  // K/V tiles taken so far, in the producer's order
        auto issue_s = [&](int j) -> bool {
            const int slot = t % C::NSLOTS;
            if (!mbar_wait(full0 + 8 * slot, (t / C::NSLOTS) & 1, give_up)) return false;
            tc_fence_after();
            const uint32_t k_addr = smem_u32(slots + slot * C::SLOT_BYTES);
#pragma unroll
            for (int ks = 0; ks < HD / 16; ++ks) {
                const uint64_t a = smem_desc_sw128(smem_u32(q_s) + (ks / 4) * C::BLOCK_BYTES) + 2 * (ks % 4);
                const uint64_t b = smem_desc_sw128_groups(k_addr + (ks / 4) * 1024, C::CB * 1024) + 2 * (ks % 4);
                umma_bf16(tmem_base + (j & 1) * AK, a, b, idesc_s, ks > 0 ? 1u : 0u);
            }
            umma_commit(empty0 + 8 * slot);       // K_j may be overwritten when these have read it
            umma_commit(s_full0 + 8 * (j & 1));
            ++t;
            return true;
        };
        if (ok && ntiles > 0) ok = issue_s(0);
        if (ok && ntiles > 1) ok = issue_s(1);
        for (int j = 0; j < ntiles && ok; ++j) {
            ok = mbar_wait(p_full0 + 8 * (j & 1), (j >> 1) & 1, give_up);
            if (!ok) break;
            const int slot = t % C::NSLOTS;
            ok = mbar_wait(full0 + 8 * slot, (t / C::NSLOTS) & 1, give_up);
            if (!ok) break;
            tc_fence_after();
            const uint32_t v_addr = smem_u32(slots + slot * C::SLOT_BYTES);
#pragma unroll
            for (int kk = 0; kk < AK / 16; ++kk) {
                // P_j lies in tensor memory where S_j was (8 columns per 16 keys)
                // keys 16 kk .. +15: rows r .. r+15 of page pg (pages of 8 tokens: both groups of 8 are whole pages)
                const int pg = (16 * kk) >> p.page_shift, r = (16 * kk) & (p.page_size - 1);
                const uint64_t b = smem_desc_mn_sw128(v_addr + (pg * C::CB * p.page_size + r) * 128, p.page_size * 128,
                                                      p.page_size >= 16 ? 1024 : C::CB * 1024);
                umma_bf16_a_tmem(tmem_base + C::O_COL + (j & 1) * HD, tmem_base + (j & 1) * AK + 8 * kk, b, idesc_o,
                                 (j >= 2 || kk > 0) ? 1u : 0u);
            }
            umma_commit(empty0 + 8 * slot);
            umma_commit(o_full0 + 8 * (j & 1));   // O of this set holds its tiles up to j
            ++t;
            // S of tile j+2 goes where S and then P of tile j were: behind PV_j in the tensor pipe
            if (j + 2 < ntiles) ok = issue_s(j + 2);
        }
    } else if (warp >= 2) {
        // ---- softmax warps: two sets, each with two threads per query row ------------------------------
        // Set 0 (warps 2..9) takes the even tiles, set 1 (warps 10..17) the odd ones, each with its own S
        // buffer, P buffer, O accumulator and row statistics (two independent online softmaxes, merged
        // at the end), so that one set's exponentials run beside the other's passes over S.  Within a
        // set, warps w and w + 4 own the same 32 TMEM lanes; `half` says which half of S's 128 columns
        // and of O's HD columns a thread works on.  The two exchange their partial row maxima through
        // shared memory once per tile; sums stay partial until the end.
        const int set = (warp - 2) >> 3;
        const int quarter = warp & 3;
        const int half = ((warp - 2) & 7) >> 2;
        const int row = quarter * 32 + lane;
        constexpr int SC = AK / 2;   // S columns per thread
        constexpr int OC = HD / 2;   // O columns per thread
        const uint32_t lane_addr = tmem_base + ((uint32_t)(quarter * 32) << 16);
        const int qp = pos0 + row;                                     // this row's position
        const int lo = p.window > 0 ? max(0, qp + 1 - p.window) : 0;   // its first visible key
        const float scale_log2 = p.scale * 1.4426950408889634f;        // softmax in base 2
        const int pair_bar = 1 + 4 * set + quarter;                    // named barrier of the 64 threads of a quarter
        float* my_x = xchg + (2 * set + half) * AQ + row;              // where the partner reads this thread's value
        float* partner_x = xchg + (2 * set + (half ^ 1)) * AQ + row;
        const uint32_t s_addr = lane_addr + set * AK + half * SC;
        const uint32_t o_set = lane_addr + C::O_COL + set * HD + half * OC;
        float m_used = -INFINITY, l_run = 0.f;  // m_used: the maximum this row's exponentials are taken against
        bool ok = true;
        for (int j = set; j < ntiles; j += 2) {
            const int tile0 = tile_lo + j * AK;
            const int col0 = tile0 + half * SC;  // position of this thread's first key
            ok = mbar_wait(s_full0 + 8 * set, (j >> 1) & 1, give_up);
            ok = __all_sync(0xffffffffu, ok);  // one decision per warp: the TMEM accesses below are warp-wide
            // tiles wholly visible to all 128 rows skip the per-element test
            const bool all_visible = tile0 + AK - 1 <= pos0 && (p.window <= 0 || tile0 > pos0 + AQ - 1 - p.window);
            // this thread's half row of S, read from TMEM once and held in registers
            float sv[SC];
            if (ok) {
                tc_fence_after();
#pragma unroll
                for (int c = 0; c < SC / 32; ++c) tmem_ld32(s_addr + 32 * c, sv + 32 * c);
                if (!all_visible) {
#pragma unroll
                    for (int i = 0; i < SC; ++i) {
                        const int pos = col0 + i;
                        sv[i] = (pos <= qp && pos >= lo) ? sv[i] : -INFINITY;
                    }
                }
                float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};  // four chains: ILP for the few warps of a scheduler
#pragma unroll
                for (int i = 0; i < SC; ++i) mx4[i & 3] = fmaxf(mx4[i & 3], sv[i]);
                *my_x = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
            }
            // (both threads of a row take every decision to leave together: their barriers stay paired)
            ok = bar_and(pair_bar, 64, ok);
            if (!ok) break;
            const float mx = fmaxf(*my_x, *partner_x);
            // The maximum moves only when a tile exceeds it by more than LAZY_STEP: exponentials up to
            // 2^LAZY_STEP are as exact in bfloat16 and float32 as those up to 1, and the accumulated O
            // (in tensor memory) then needs rescaling for the first tiles of a row at most.
            const float m_tile = mx * scale_log2;
            float alpha = 1.f;
            bool rescale = false;
            if (m_tile > m_used + LAZY_STEP) {  // (false for a tile without a visible key: -inf)
                if (m_used != -INFINITY) {
                    alpha = ex2(m_used - m_tile);
                    rescale = true;
                }
                m_used = m_tile;
            }
            const float base = (m_used == -INFINITY) ? 0.f : m_used;
            // P goes to this set's buffer, last read by PV of the set's previous tile; when that is
            // complete, O of the set is at rest as well (for the rescaling below)
            if (j >= 2) {
                ok = mbar_wait(o_full0 + 8 * set, ((j - 2) >> 1) & 1, give_up);
                ok = __all_sync(0xffffffffu, ok);
            }
            ok = bar_and(pair_bar, 64, ok);  // (also: the partner has read this thread's maximum)
            if (!ok) break;
            float sum4[4] = {0.f, 0.f, 0.f, 0.f};
            // P as the second MMA's A operand, in tensor memory over the first quarter of this set's S
            // (which both threads of the row hold in registers by now): pairs of keys per column
#pragma unroll
            for (int c = 0; c < SC / 32; ++c) {
                float* v = sv + 32 * c;
                // straight-line code, so that the 32 exponentials are in flight together; 2^-inf is exactly 0
#pragma unroll
                for (int i = 0; i < 32; ++i) v[i] = ex2(fmaf(v[i], scale_log2, -base));
#pragma unroll
                for (int i = 0; i < 32; ++i) sum4[i & 3] += v[i];
                float packed[16];
#pragma unroll
                for (int i = 0; i < 16; ++i) packed[i] = __uint_as_float(pack2(v[2 * i], v[2 * i + 1]));
                tmem_st16(lane_addr + set * AK + half * (SC / 2) + 16 * c, packed);
            }
            l_run = l_run * alpha + ((sum4[0] + sum4[1]) + (sum4[2] + sum4[3]));
            if (__any_sync(0xffffffffu, rescale)) {
                // O of this set so far times alpha, row by row, before PV of this tile adds to it: the
                // MMA warp waits for every thread's arrival below
                tc_fence_after();
                rescale_o<OC>(o_set, alpha);
            }
            tc_fence_before();
            asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(p_full0 + 8 * set) : "memory");
        }
        // ---- the row's sum over both halves; every thread comes here, whatever happened above ----------
        *my_x = l_run;
        asm volatile("bar.sync %0, 64;" ::"r"(pair_bar) : "memory");
        l_run += *partner_x;
        asm volatile("bar.sync %0, 64;" ::"r"(pair_bar) : "memory");
        // this set's last PV
        const int my_tiles = ntiles > set ? (ntiles - set + 1) / 2 : 0;
        if (ok && my_tiles > 0) {
            ok = mbar_wait(o_full0 + 8 * set, (my_tiles - 1) & 1, give_up);
            ok = __all_sync(0xffffffffu, ok);
        }
        // ---- the two sets merge: set 1 leaves (m, l) per row, set 0 reads both accumulators -------------
        // (in the two exchange slots of set 1's own row, at rest after the pair's barriers above)
        float* set1_m = xchg + 2 * AQ + row;
        float* set1_l = xchg + 3 * AQ + row;
        if (set == 1 && half == 0) {
            *set1_m = m_used;
            *set1_l = l_run;
        }
        tc_fence_before();
        ok = bar_and(9, 512, ok);
        if (set == 0) {
            tc_fence_after();
            const float m1 = *set1_m, l1 = *set1_l;
            const float M = fmaxf(m_used, m1);
            const float w0 = (m_used == -INFINITY) ? 0.f : ex2(m_used - M);
            const float w1 = (m1 == -INFINITY) ? 0.f : ex2(m1 - M);
            const float L = w0 * l_run + w1 * l1;
            const uint32_t o_addr0 = lane_addr + C::O_COL + half * OC, o_addr1 = o_addr0 + HD;
            // a half row of the merged, unnormalised O, 32 columns at a time (an accumulator that no tile went into is not read)
            auto merged = [&](int c, float* v) {
                float u[32];
                if (ntiles > 0) {
                    tmem_ld32(o_addr0 + 32 * c, v);
                } else {
#pragma unroll
                    for (int i = 0; i < 32; ++i) v[i] = 0.f;
                }
                if (ntiles > 1) {
                    tmem_ld32(o_addr1 + 32 * c, u);
#pragma unroll
                    for (int i = 0; i < 32; ++i) v[i] = fmaf(w1, u[i], w0 * v[i]);
                } else {
#pragma unroll
                    for (int i = 0; i < 32; ++i) v[i] *= w0;
                }
            };
            bf16* o = p.out + ((size_t)(row0 + q0 + row) * p.nh + h) * HD + half * OC;
            if (parts == 1) {
                if (ok) {
                    const float inv = L > 0.f ? 1.f / L : 0.f;
#pragma unroll
                    for (int c = 0; c < OC / 32; ++c) {
                        float v[32];
                        merged(c, v);
                        if (row < nq) {
#pragma unroll
                            for (int q4 = 0; q4 < 4; ++q4) {
                                uint4 w;
                                w.x = pack2(v[8 * q4 + 0] * inv, v[8 * q4 + 1] * inv);
                                w.y = pack2(v[8 * q4 + 2] * inv, v[8 * q4 + 3] * inv);
                                w.z = pack2(v[8 * q4 + 4] * inv, v[8 * q4 + 5] * inv);
                                w.w = pack2(v[8 * q4 + 6] * inv, v[8 * q4 + 7] * inv);
                                *reinterpret_cast<uint4*>(o + 32 * c + 8 * q4) = w;
                            }
                        }
                    }
                }
            } else {
                // ---- one part of a cut row of keys: leave (m, l, unnormalised O), the last part to arrive merges ----
                // part_o is [item][head][column][row]: a warp's 32 rows lie side by side, so that its stores
                // here and its loads in the merge are whole 128-byte lines
                float* my_o = p.part_o + (((size_t)item * p.nh + h) * HD + half * OC) * AQ + row;
                float* my_ml = p.part_ml + (((size_t)item * p.nh + h) * AQ + row) * 2;
#pragma unroll
                for (int c = 0; c < OC / 32; ++c) {
                    float v[32];
                    if (ok) {
                        merged(c, v);
                    } else {
#pragma unroll
                        for (int i = 0; i < 32; ++i) v[i] = 0.f;
                    }
#pragma unroll
                    for (int i = 0; i < 32; ++i) my_o[(32 * c + i) * AQ] = v[i];
                }
                if (half == 0) {
                    my_ml[0] = M;
                    my_ml[1] = L;
                }
                // Release / acquire through the counter: the barrier orders every thread's stores before
                // thread 64's release, and its acquire before every thread's loads of the other parts.
                asm volatile("bar.sync 10, 256;" ::: "memory");
                if (tid == 64) {
                    int* counter = p.counters + (size_t)first_item * p.nh + h;
                    int prev;
                    asm volatile("atom.add.acq_rel.gpu.global.s32 %0, [%1], 1;" : "=r"(prev) : "l"(counter) : "memory");
                    *last_part = (prev == parts - 1);
                    if (prev == parts - 1) *counter = 0;  // ready for the next launch
                }
                asm volatile("bar.sync 10, 256;" ::: "memory");
                if (*last_part && row < nq) {
                    // every load of a round is in flight before the first is used: the (m, l) of all parts,
                    // then O in rounds of 16 or 8 columns of KP parts each (in part order whoever came last)
                    const size_t stride_o = (size_t)p.nh * AQ * HD, stride_ml = (size_t)p.nh * AQ * 2;
                    const float* ml0 = p.part_ml + (((size_t)first_item * p.nh + h) * AQ + row) * 2;
                    const float* o0 = p.part_o + (((size_t)first_item * p.nh + h) * HD + half * OC) * AQ + row;
                    float2 ml[PREFILL_MAX_PARTS];
#pragma unroll
                    for (int k = 0; k < PREFILL_MAX_PARTS; ++k)
                        ml[k] = k < parts ? *reinterpret_cast<const float2*>(ml0 + k * stride_ml) : make_float2(-INFINITY, 0.f);
                    float Mp = -INFINITY, Lp = 0.f, wk[PREFILL_MAX_PARTS];
#pragma unroll
                    for (int k = 0; k < PREFILL_MAX_PARTS; ++k) Mp = fmaxf(Mp, ml[k].x);
#pragma unroll
                    for (int k = 0; k < PREFILL_MAX_PARTS; ++k) {
                        wk[k] = (ml[k].x == -INFINITY) ? 0.f : ex2(ml[k].x - Mp);
                        Lp = fmaf(wk[k], ml[k].y, Lp);
                    }
                    const float inv = Lp > 0.f ? 1.f / Lp : 0.f;
                    auto merge = [&](auto kp_tag) {
                        constexpr int KP = decltype(kp_tag)::value;            // parts unrolled (2, 4 or 8)
                        constexpr int F = KP >= 4 ? 8 : 16;                    // columns per round
#pragma unroll 1
                        for (int c0 = 0; c0 < OC; c0 += F) {
                            float v[KP][F];
#pragma unroll
                            for (int k = 0; k < KP; ++k)
#pragma unroll
                                for (int i = 0; i < F; ++i) v[k][i] = k < parts ? o0[k * stride_o + (size_t)(c0 + i) * AQ] : 0.f;
#pragma unroll
                            for (int i = 0; i < F; i += 8) {
                                float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
                                for (int k = 0; k < KP; ++k)
#pragma unroll
                                    for (int e = 0; e < 8; ++e) acc[e] = fmaf(wk[k], v[k][i + e], acc[e]);
                                uint4 w;
                                w.x = pack2(acc[0] * inv, acc[1] * inv);
                                w.y = pack2(acc[2] * inv, acc[3] * inv);
                                w.z = pack2(acc[4] * inv, acc[5] * inv);
                                w.w = pack2(acc[6] * inv, acc[7] * inv);
                                *reinterpret_cast<uint4*>(o + c0 + i) = w;
                            }
                        }
                    };
                    if (parts <= 2) merge(std::integral_constant<int, 2>{});
                    else if (parts <= 4) merge(std::integral_constant<int, 4>{});
                    else merge(std::integral_constant<int, 8>{});
                }
            }
        }
    }
    __syncwarp();
    if (*give_up && tid == 0) cw_report(p.status, CW_ST_WAIT_TIMEOUT, blockIdx.x, blockIdx.y);
    tc_fence_before();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem_base, C::TMEM_COLS);
}

// ---------------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------------
template <int HD>
static int launch_prefill_tc(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv,
                             const PrefillTcParams& p, int items, cudaStream_t stream) {
    using C = ACfg<HD>;
    static bool configured = false;
    if (!configured) {
        if (cudaFuncSetAttribute(attn_prefill_tc_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 C::SMEM_BYTES) != cudaSuccess)
            return (int)cudaGetLastError();
        configured = true;
    }
    return cw_launch(attn_prefill_tc_kernel<HD>, dim3(p.nh, items), dim3(A_THREADS), C::SMEM_BYTES, stream, 1, mq, mk, mv, p);
}

// q: [q_rows, q_cols] rows of the flat batch (row stride q_stride, head h at columns h*hd..), out:
// [q_rows, nh*hd]; item_seq/item_q0: one entry per 128 query rows of each request, or several (parts
// of its keys, see PrefillTcParams::item_split; then part_o holds items * nh * 128 * hd floats, part_ml
// items * nh * 256 and counters items * nh zeros, which the kernel leaves zero).  Takes head sizes
// 64 and 128 and pages of 8..128 tokens (a power of two); CW_ERR_UNSUPPORTED otherwise, so that the
// caller can use the mma.sync kernel.
extern "C" int cw_attention_prefill_tc(const void* q, int q_stride, int q_cols, int q_rows, void* out,
                                       const void* k_cache, const void* v_cache, const int* block_tables,
                                       const int* q_start, const int* ctx_lens, const int* item_seq,
                                       const int* item_q0, const int* item_split, float* part_o, float* part_ml,
                                       int* counters, int items, int nh, int nkv, int hd, int page_size,
                                       int max_blocks, int num_pages, float scale, int window, int* status,
                                       cudaStream_t stream) {
    if (items == 0) return CW_OK;
    if (items < 0 || nh <= 0 || nkv <= 0 || nh % nkv != 0 || page_size <= 0 || max_blocks <= 0 || num_pages <= 0 ||
        q_rows <= 0 || q_cols < nh * hd)
        return CW_ERR_BAD_SIZE;
    if (item_split != nullptr && (part_o == nullptr || part_ml == nullptr || counters == nullptr)) return CW_ERR_BAD_SIZE;
    if (hd != 64 && hd != 128) return CW_ERR_UNSUPPORTED;
    if ((page_size & (page_size - 1)) != 0 || page_size < 8 || page_size > AK) return CW_ERR_UNSUPPORTED;
    if (q_stride % 8 != 0 || ((uintptr_t)q & 15) || ((uintptr_t)k_cache & 15) || ((uintptr_t)v_cache & 15) ||
        ((uintptr_t)out & 15))
        return CW_ERR_UNSUPPORTED;
    if (nh > 65535 || items > 65535) return CW_ERR_BAD_SIZE;
    if (load_encode() != 0) return CW_ERR_UNSUPPORTED;
    CUtensorMap mq, mk, mv;
    {
        const cuuint64_t dims[2] = {(cuuint64_t)q_cols, (cuuint64_t)q_rows};
        const cuuint64_t strides[1] = {(cuuint64_t)q_stride * 2};
        const cuuint32_t box[2] = {64, AQ};
        const cuuint32_t elem[2] = {1, 1};
        if (g_encode(&mq, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(q), dims, strides, box, elem,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
            return CW_ERR_UNSUPPORTED;
    }
    {
        // K: the cache as [64 elements][8 slots][64-element block][groups of 8 slots][kv head]: a box is one page
        // of one head, landing as [group][block][8 tokens][128 bytes]
        const cuuint64_t row = (cuuint64_t)nkv * hd * 2;
        const cuuint64_t dims[5] = {64, 8, (cuuint64_t)(hd / 64), (cuuint64_t)num_pages * page_size / 8, (cuuint64_t)nkv};
        const cuuint64_t strides[4] = {row, 128, 8 * row, (cuuint64_t)hd * 2};
        const cuuint32_t box[5] = {64, 8, (cuuint32_t)(hd / 64), (cuuint32_t)(page_size / 8), 1};
        const cuuint32_t elem[5] = {1, 1, 1, 1, 1};
        if (g_encode(&mk, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 5, const_cast<void*>(k_cache), dims, strides, box, elem,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
            return CW_ERR_UNSUPPORTED;
    }
    {
        // V: the same memory as [64 elements][slot][64-element block][kv head]: a box is one page of one head with
        // all its blocks, which land one after the other ([block][token][128 bytes])
        const cuuint64_t dims[4] = {64, (cuuint64_t)num_pages * page_size, (cuuint64_t)(hd / 64), (cuuint64_t)nkv};
        const cuuint64_t strides[3] = {(cuuint64_t)nkv * hd * 2, 128, (cuuint64_t)hd * 2};
        const cuuint32_t box[4] = {64, (cuuint32_t)page_size, (cuuint32_t)(hd / 64), 1};
        const cuuint32_t elem[4] = {1, 1, 1, 1};
        if (g_encode(&mv, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(v_cache), dims, strides, box, elem,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
            return CW_ERR_UNSUPPORTED;
    }
    PrefillTcParams p;
    p.out = (bf16*)out;
    p.block_tables = block_tables; p.q_start = q_start; p.ctx_lens = ctx_lens;
    p.item_seq = item_seq; p.item_q0 = item_q0;
    p.item_split = item_split; p.part_o = part_o; p.part_ml = part_ml; p.counters = counters;
    p.nh = nh; p.nkv = nkv; p.page_size = page_size; p.page_shift = __builtin_ctz(page_size);
    p.max_blocks = max_blocks; p.num_pages = num_pages;
    p.scale = scale; p.window = window; p.status = status;
    return hd == 64 ? launch_prefill_tc<64>(mq, mk, mv, p, items, stream) : launch_prefill_tc<128>(mq, mk, mv, p, items, stream);
}

CW_TRACE_TU(attention_prefill_tc)
