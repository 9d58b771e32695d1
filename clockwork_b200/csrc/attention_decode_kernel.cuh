// Paged decode attention in bfloat16: every request brings one query token and reads its whole
// context from the cache.  The step is a stream of K/V pages from HBM, so the context of a request
// is split over CTAs and all query heads of one KV head share each K/V tile.  The split size is a
// run-time value (a multiple of 64, at least 128): with few requests the context is cut finely so
// that every SM has a CTA; with many requests a CTA walks a whole context and nothing is merged.
// A CTA runs its code once, so the kernel is written for a small instruction footprint (one-shot
// loops are not unrolled, divisions are out of line, the split merge is one compact form).
//
// Reference: clockwork/kernels/attention.py:113-134 (masking keys >= ctx_len, softmax, P.V) and the
// Triton kernel clockwork/kernels/triton_paged_attn.py:16-106 (online softmax over one page per
// iteration, float32 accumulation).  That kernel runs one program per (sequence, query head), so
// every query head re-reads its KV head (:49); here a CTA is (KV head, sequence, context split), the
// group's query heads are the 16 rows of a tensor-core tile (mma.sync m16n8k16), and the splits are
// merged by the CTA that finishes last, in split order.
//
// Scores, softmax and accumulation are float32; probabilities are rounded to bfloat16 for P.V.
//
// How the splits of a (request, KV head) group meet, two forms.  Through global memory (the usual one):
// partials and log-sum-exps go to a float32 workspace and the CTA that arrives last at the group's
// counter merges them, in split order; more than 36 splits meet in two levels (twelve splits share a
// counter, the last of them merges the twelve, the last of these mergers merges their results).
// Through a thread-block cluster (on request, up to 16 splits): the splits of a group are the CTAs of
// one cluster; each pushes its normalised partial output, cut into as many slices as there are
// splits, into the others' shared memory (slice j to CTA j) with its log-sum-exps, arrives on their
// barriers, waits for theirs, and merges and stores its own slice, sources in split order: no global
// scratch, no counter, no second pass by one CTA; measured slower inside a step, because a cluster
// starts only when all of its CTAs find room at once.
#pragma once
#include "attention_mma.cuh"
#include "tc_common.cuh"

#define MAX_CLUSTER 16

__device__ __forceinline__ uint32_t peer_smem(uint32_t local_addr, uint32_t rank) {
    uint32_t remote;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local_addr), "r"(rank));
    return remote;
}
__device__ __forceinline__ void cluster_barrier() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}

#define TILE 64
#define MIN_SPLIT 128  // smallest context split (tokens per CTA); the grid's z extent is sized for it
#define NWARPS 4

struct DecodeParams {
    const bf16* q; int q_stride;
    bf16* out;
    const bf16* k_cache; const bf16* v_cache;
    const int* block_tables; const int* ctx_lens;
    const int* q_start;  // null: request s owns row s of q and out.  Else [S + 1]: request s owns rows q_start[s] ..
                         // q_start[s + 1] of a flat batch; only requests with exactly one row are served here
    int nh, nkv, qgroups, page_size, page_shift, max_blocks, num_pages;
    float scale; int window;
    float* part_o;   // [S, nh, max_splits, HD]
    float* part_lse; // [S, nh, max_splits]
    int max_splits;
    int split;            // tokens per CTA, used when split_ptr is null
    const int* split_ptr; // the same on the device (so that a captured graph can change it per step)
    int max_split_pages;  // page ids a split may need (sizes the shared-memory page list)
    int stages;           // tiles in flight per CTA: 4 (default) or 2
    int swizzle;          // with 2 tiles in flight: the unpadded, swizzled K/V layout (three CTAs per SM)
    int tma;              // K/V tiles arrive as one TMA copy per page and operand (head sizes of 64n, pages of 8..64 tokens)
    int tree;             // the variant that merges more than 36 splits in two levels (two tiles in flight, no cluster)
    int cluster;          // > 1: the grid's z extent is one cluster of this many CTAs and the splits meet through it
    int max_ctx;          // the bound on every context that sized the grid
    int* counters;   // [S * nkv * qgroups]
    int* status;
    // Fused position encoding and cache write (kv_new != null): q, and the new token's k and v, are
    // taken raw from the [q | k | v] rows; q and k are rotated here, k and v stored at slots[s].
    const bf16* kv_new;      // the [q | k | v] rows (row stride q_stride), or null
    const float* inv_freq;   // [rotary_dim / 2] or null (no rotation)
    int rotary_dim;
    const int* slots;        // [S] cache slot of the new token (-1: not stored)
    bf16* k_cache_w; bf16* v_cache_w;
    int num_slots;
};

__device__ __forceinline__ void cp_async_wait_upto(int n) {
    switch (n) {
        case 0: cp_async_wait<0>(); break;
        case 1: cp_async_wait<1>(); break;
        case 2: cp_async_wait<2>(); break;
        default: cp_async_wait<3>(); break;
    }
}

__device__ __forceinline__ bool mine_newest(int newest, int t0, int t1, int kv_begin) {
    return newest >= t0 && newest < t1 && newest >= kv_begin;
}

// ST: tiles in flight.  4 puts a whole split (256 tokens) in flight at once, for steps with few
// CTAs where latency is everything; 2 halves the shared memory so that two CTAs share an SM.
// Position -> (block, offset) for page sizes that are no power of two: out of line, so that the
// division's instruction sequence exists once in the kernel instead of at every use.
static __device__ __noinline__ int2 block_and_offset(int pos, int page_size) { return make_int2(pos / page_size, pos % page_size); }

__device__ __forceinline__ void tma_page_4d(uint32_t dst, const CUtensorMap* map, int x, int y, int z, int w, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
        ::"r"(dst), "l"(map), "r"(bar), "r"(x), "r"(y), "r"(z), "r"(w)
        : "memory");
}

// LAYOUT: how a K/V tile lies in shared memory and how it gets there (see the kernel's first lines).
#define KV_PADDED 0
#define KV_SWIZZLED 1
#define KV_TMA 2

template <int HD, int ST, int LAYOUT, bool CL, bool TREE>
__global__ void __launch_bounds__(NWARPS * 32)
attn_decode_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v, const DecodeParams p) {
    constexpr int LD = HD + 8;  // padded q row (elements): consecutive rows fall into different banks
    // K/V tiles, three layouts.  Padded rows (as for q): plain addressing, the smallest instruction count,
    // for steps with few CTAs.  Swizzled (head sizes that are multiples of 64): unpadded rows with their
    // 16-byte chunks XOR-swizzled by the row (chunk c of row r lies at chunk c ^ (r & 7)), as free of
    // bank conflicts and small enough for three CTAs per SM, for steps with many CTAs.  Both are filled
    // by 16-byte cp.async, 2,048 of them per tile.  TMA (the same head sizes, pages of 8 to 64 tokens): a
    // tile lies page by page, [page][64-column block][token][128 bytes] with the hardware's 128-byte
    // swizzle (the same XOR, within a block), and one warp fetches it with one copy per page and
    // operand, completion counted by an mbarrier per stage; rows that no visible key owns arrive with
    // whatever the pages hold and are masked (scores) or cleared (values) in shared memory.
    constexpr bool TMA = LAYOUT == KV_TMA;
    constexpr bool SWZ = LAYOUT != KV_PADDED && HD % 64 == 0;
    static_assert(!TMA || HD % 64 == 0, "TMA tiles are made of 64-column blocks");
    constexpr int LDK = SWZ ? HD : HD + 8;
    constexpr int CB = HD / 64;
    const int ps_shift = p.page_shift;
    auto kv_off = [&](int r, int c) -> int {
        if (TMA)
            return (((((r >> ps_shift) * CB + (c >> 3)) << ps_shift) + (r & (p.page_size - 1))) << 6) + (((c & 7) ^ (r & 7)) << 3);
        return r * LDK + (SWZ ? ((c ^ (r & 7)) << 3) : (c << 3));
    };
    // (the swizzled TMA tiles need a 1024-byte aligned base: they come first, and the kernel checks)
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    bf16* Qs = TMA ? (bf16*)smem_raw + 2 * ST * TILE * LDK : (bf16*)smem_raw;   // [16][LD]
    bf16* Ks = TMA ? (bf16*)smem_raw : Qs + 16 * LD;                            // [ST][TILE][LDK]
    bf16* Vs = Ks + ST * TILE * LDK;                                            // [ST][TILE][LDK]
    int* page_s = (int*)((TMA ? Qs : Vs + ST * TILE * LDK) + (TMA ? 16 * LD : 0));  // [max_split_pages] page of every block of this split
    __shared__ __align__(8) unsigned long long full_bar[TMA ? ST : 1];  // TMA: the copies of a stage have landed
    __shared__ int give_up;
    __shared__ float ml_s[NWARPS][16][2];
    __shared__ float w_s[16][16];               // final merge: weight of each split per query row
    __shared__ __align__(16) bf16 new_s[2 * HD]; // the newest token's k and v
    __shared__ float cs_s[HD];                  // cos, sin of the newest position (fused rotation)
    __shared__ int last_flag;
    // cluster merge: the slices of this CTA's share that the splits of the group push here, by source
    // (a source's slice is `quota` groups of four outputs), their log-sum-exps, and the barrier they arrive on
    __shared__ float4 inbox_s[CL ? 16 * HD / 4 + MAX_CLUSTER : 1];
    __shared__ float lse_all[CL ? MAX_CLUSTER : 1][16];
    __shared__ __align__(8) unsigned long long merge_bar;

    // Nothing below reads what the preceding kernels of this step wrote until pdl_wait(): context
    // lengths, block tables, positions and the split size are inputs of the step, and cached keys and
    // values of earlier tokens were written by earlier steps.  So the page list and the first tiles
    // are fetched while the preceding kernel finishes; only q and the newest token's k/v come after.
    pdl_launch_dependents();
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, t = lane & 3;
    const int kvh = blockIdx.x / p.qgroups, qg = blockIdx.x % p.qgroups;
    const int s = blockIdx.y, sp = blockIdx.z;
    const int G = p.nh / p.nkv;
    const int h0 = kvh * G + qg * 16;
    const int rows = min(16, G - qg * 16);
    int row = s;  // the request's row in q, kv_new, slots and out
    bool mine = true;
    if (p.q_start != nullptr) {
        row = p.q_start[s];
        mine = p.q_start[s + 1] - row == 1;  // (a prompt portion is the prefill kernel's work)
    }
    const int ctx = mine ? p.ctx_lens[s] : 0;
    int SPLIT = p.split_ptr != nullptr ? *p.split_ptr : p.split;
    if (CL) {
        // no more splits than the cluster has CTAs, whatever the step's policy asked for
        const int least = ((p.max_ctx + p.cluster - 1) / p.cluster + TILE - 1) / TILE * TILE;
        SPLIT = max(SPLIT, least);
    }
    const int kv_begin = p.window > 0 ? max(0, ctx - p.window) : 0;
    const int nsplits = ctx > 0 ? (ctx + SPLIT - 1) / SPLIT : 0;
    const int first_split = kv_begin / SPLIT;
    const int active = nsplits - first_split;  // the splits of this group that have keys
    if (CL) {
        // Every CTA of the cluster, also one with nothing to do, passes this barrier; behind it the
        // barriers that the group's splits arrive on exist, each expecting the other active splits.
        if (tid == 0) {
            asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_addr(&merge_bar)), "r"(max(1, active - 1)) : "memory");
            asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        }
        cluster_barrier();
    }
    if (!mine) return;
    if (ctx <= 0) {  // a padding row of a fixed-shape batch
        pdl_wait();
        if (sp == 0)
            for (int i = tid; i < rows * HD; i += blockDim.x)
                p.out[((size_t)row * p.nh + h0 + i / HD) * HD + i % HD] = __float2bfloat16_rn(0.f);
        return;
    }
    if (sp < first_split || sp >= nsplits) return;  // (no end record: these CTAs do nothing)
    const int t0 = sp * SPLIT, t1 = min(ctx, t0 + SPLIT);
    const int* table = p.block_tables + (size_t)s * p.max_blocks;
    const float scale_log2 = p.scale * 1.4426950408889634f;  // softmax in base 2: exp(x) = 2^(x log2 e)

    if (TMA) {
        if (smem_addr(smem_raw) & 1023) {
            if (tid == 0) cw_report(p.status, CW_ST_SMEM_ALIGN, blockIdx.x, (int)(smem_addr(smem_raw) & 1023));
            return;
        }
        if (tid == 0) {
            for (int i = 0; i < ST; ++i) mbar_init(smem_addr(&full_bar[i]), 1);
            give_up = 0;
            asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        }
        if (warp == 0 && lane < 2) asm volatile("prefetch.tensormap [%0];" ::"l"(lane == 0 ? &map_k : &map_v) : "memory");
    }
    // page ids of the split's blocks, looked up once: tile loads then depend on shared memory only
    const int blk0 = p.page_shift >= 0 ? t0 >> p.page_shift : t0 / p.page_size;
    const int blk1 = p.page_shift >= 0 ? (t1 - 1) >> p.page_shift : (t1 - 1) / p.page_size;
    if ((min(SPLIT, p.max_ctx) + p.page_size - 1) / p.page_size + 1 > p.max_split_pages) {
        // The split read from the device is longer than the bound that sized the page list.  The test
        // is the same in every CTA of the launch: all of them leave, and no group's counter is touched.
        if (tid == 0) cw_report(p.status, CW_ST_SPLIT_BOUND, s, SPLIT);
        return;
    }
    for (int i = tid; i <= blk1 - blk0 && i < p.max_split_pages; i += blockDim.x) {
        const int blk = blk0 + i;
        int page = blk < p.max_blocks ? table[blk] : -1;
        if (page >= p.num_pages) page = -1;
        if (page < 0 && (blk + 1) * p.page_size > kv_begin) cw_report(p.status, CW_ST_PAGE_RANGE, s, page);
        page_s[i] = page;
    }
    __syncthreads();  // page_s visible

    // Every thread copies the same 16-byte column of several rows: the row's cache slot is worked
    // out once per row and the rest of the addressing is compile-time strides.
    constexpr int CH = HD / 8;                                  // 16-byte chunks per row
    constexpr bool EVEN = (NWARPS * 32) % CH == 0;              // threads split evenly over a row's chunks
    constexpr int RPP = EVEN ? (NWARPS * 32) / CH : 1;          // rows per pass
    const int newest = ctx - 1;  // its k/v are written by this step: they arrive after pdl_wait()
    auto slot_of = [&](int pos) -> int {
        if (pos >= t1 || pos < kv_begin || pos == newest) return -1;
        int blk, off;
        if (p.page_shift >= 0) {
            blk = pos >> p.page_shift;
            off = pos & (p.page_size - 1);
        } else {
            const int2 bo = block_and_offset(pos, p.page_size);
            blk = bo.x;
            off = bo.y;
        }
        const int page = blk - blk0 < p.max_split_pages ? page_s[blk - blk0] : -1;
        if (page < 0) return -1;
        return page * p.page_size + off;
    };
    auto copy_chunk = [&](bf16* kd, bf16* vd, int r, int c, int slot) {
        if (slot >= 0) {
            const size_t src = ((size_t)slot * p.nkv + kvh) * HD + c * 8;
            cp_async16(kd + kv_off(r, c), p.k_cache + src);
            cp_async16(vd + kv_off(r, c), p.v_cache + src);
        } else {
            *reinterpret_cast<uint4*>(kd + kv_off(r, c)) = make_uint4(0, 0, 0, 0);
            *reinterpret_cast<uint4*>(vd + kv_off(r, c)) = make_uint4(0, 0, 0, 0);
        }
    };
    auto load_tile = [&](int tile_idx) {
        bf16* kd = Ks + (tile_idx % ST) * TILE * LDK;
        bf16* vd = Vs + (tile_idx % ST) * TILE * LDK;
        const int pos0 = t0 + tile_idx * TILE;
        if (TMA) {
            // lanes 0 .. pages-1 of warp 0 fetch the K pages of the tile, the next lanes its V pages; a
            // page that the split does not own (past its end, or dropped behind the window) is read
            // from page 0: nothing of it is used
            if (warp == 0) {
                const int pages = TILE >> ps_shift;
                const uint32_t bar = smem_addr(&full_bar[tile_idx % ST]);
                if (lane == 0) mbar_expect_tx(bar, 2 * TILE * HD * 2);
                __syncwarp();
                if (lane < 2 * pages) {
                    const bool is_v = lane >= pages;
                    const int j = is_v ? lane - pages : lane;
                    const int i = (pos0 >> ps_shift) + j - blk0;
                    int page = (i <= blk1 - blk0 && i < p.max_split_pages) ? page_s[i] : 0;
                    if (page < 0) page = 0;
                    // what this stage held was read, and in places written, by ordinary loads and stores
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                    tma_page_4d(smem_addr((is_v ? vd : kd) + ((j * CB) << (ps_shift + 6))), is_v ? &map_v : &map_k, 0,
                                page << ps_shift, 0, kvh, bar);
                }
            }
            return;
        }
        if (EVEN) {
            const int c = tid % CH, r0 = tid / CH;
#pragma unroll 2
            for (int k = 0; k < (TILE + RPP - 1) / RPP; ++k) {
                const int r = r0 + k * RPP;
                if (r < TILE) copy_chunk(kd, vd, r, c, slot_of(pos0 + r));
            }
        } else {
            for (int i = tid; i < TILE * CH; i += blockDim.x) copy_chunk(kd, vd, i / CH, i % CH, slot_of(pos0 + i / CH));
        }
        cp_async_commit();
    };

    const int ntiles = (t1 - t0 + TILE - 1) / TILE;
#pragma unroll 1
    for (int i = 0; i < ST && i < ntiles; ++i) load_tile(i);
    // cos/sin of the new token's position (an input of the step), for the fused rotation
    const int half = p.rotary_dim >> 1;
    if (p.kv_new != nullptr && p.inv_freq != nullptr)
        for (int j = tid; j < half; j += blockDim.x) {
            const float ang = (float)newest * p.inv_freq[j];
            sincosf(ang, &cs_s[half + j], &cs_s[j]);  // one argument reduction for both
        }

    // Full rotation (the usual case): q rows and the new k are rotated on their way into shared memory,
    // each thread taking the two 16-byte chunks that pair up (elements j and j + HD/2), in one pass.
    const bool has_newest = mine_newest(newest, t0, t1, kv_begin);
    const bool rotate_on_load = p.kv_new != nullptr && p.inv_freq != nullptr && p.rotary_dim == HD && HD % 16 == 0;
    if (rotate_on_load) {
        for (int i = tid; i < (16 - rows) * CH; i += blockDim.x)  // the unused q rows of the MMA tile
            *reinterpret_cast<uint4*>(Qs + (rows + i / CH) * LD + (i % CH) * 8) = make_uint4(0, 0, 0, 0);
        __syncthreads();  // cs_s visible
    }
    pdl_wait();
    if (rotate_on_load) {
        constexpr int HC = HD / 16;  // chunk pairs per row
        const int q_units = rows * HC, k_units = has_newest ? HC : 0, v_units = has_newest ? CH : 0;
        for (int u = tid; u < q_units + k_units + v_units; u += blockDim.x) {
            if (u >= q_units + k_units) {  // the new v: a plain copy
                const int c = u - q_units - k_units;
                *reinterpret_cast<uint4*>(new_s + HD + c * 8) = *reinterpret_cast<const uint4*>(
                    p.kv_new + (size_t)row * p.q_stride + (size_t)(p.nh + p.nkv + kvh) * HD + c * 8);
                continue;
            }
            const bool is_q = u < q_units;
            const int r = is_q ? u / HC : 0, c = is_q ? u % HC : u - q_units;
            const bf16* src = is_q ? p.q + (size_t)row * p.q_stride + (size_t)(h0 + r) * HD
                                   : p.kv_new + (size_t)row * p.q_stride + (size_t)(p.nh + kvh) * HD;
            bf16* dst = is_q ? Qs + r * LD : new_s;
            uint4 lo = *reinterpret_cast<const uint4*>(src + c * 8);
            uint4 hi = *reinterpret_cast<const uint4*>(src + HD / 2 + c * 8);
            bf16* x1 = reinterpret_cast<bf16*>(&lo);
            bf16* x2 = reinterpret_cast<bf16*>(&hi);
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                const float cs = cs_s[c * 8 + e], sn = cs_s[HD / 2 + c * 8 + e];
                const float a = __bfloat162float(x1[e]), b = __bfloat162float(x2[e]);
                x1[e] = __float2bfloat16_rn(a * cs - b * sn);
                x2[e] = __float2bfloat16_rn(b * cs + a * sn);
            }
            *reinterpret_cast<uint4*>(dst + c * 8) = lo;
            *reinterpret_cast<uint4*>(dst + HD / 2 + c * 8) = hi;
        }
        __syncthreads();  // Qs and new_s visible
    } else {
    // ---- Q rows of this group into shared memory ----------------------------------------------------
    for (int i = tid; i < 16 * CH; i += blockDim.x) {
        const int r = i / CH, c = i % CH;
        uint4 v = make_uint4(0, 0, 0, 0);
        if (r < rows) v = *reinterpret_cast<const uint4*>(p.q + (size_t)row * p.q_stride + (size_t)(h0 + r) * HD + c * 8);
        *reinterpret_cast<uint4*>(Qs + r * LD + c * 8) = v;
    }
    // ---- the newest token's k and v: from the [q|k|v] row (rotating k, storing both) or from the cache
    if (has_newest) {
        if (p.kv_new != nullptr) {
            const bf16* krow = p.kv_new + (size_t)row * p.q_stride + (size_t)(p.nh + kvh) * HD;
            const bf16* vrow = p.kv_new + (size_t)row * p.q_stride + (size_t)(p.nh + p.nkv + kvh) * HD;
            for (int i = tid; i < 2 * CH; i += blockDim.x) {
                const bf16* src = (i < CH ? krow : vrow) + (i % CH) * 8;
                *reinterpret_cast<uint4*>(new_s + (i < CH ? 0 : HD) + (i % CH) * 8) = *reinterpret_cast<const uint4*>(src);
            }
        } else {
            const int blk = p.page_shift >= 0 ? newest >> p.page_shift : newest / p.page_size;
            const int page = blk - blk0 < p.max_split_pages ? page_s[blk - blk0] : -1;
            if (page >= 0) {
                const int slot = page * p.page_size + (p.page_shift >= 0 ? newest & (p.page_size - 1) : newest % p.page_size);
                const size_t src = ((size_t)slot * p.nkv + kvh) * HD;
                for (int i = tid; i < 2 * CH; i += blockDim.x)
                    *reinterpret_cast<uint4*>(new_s + (i < CH ? 0 : HD) + (i % CH) * 8) =
                        *reinterpret_cast<const uint4*>((i < CH ? p.k_cache : p.v_cache) + src + (i % CH) * 8);
            } else {
                for (int i = tid; i < 2 * HD; i += blockDim.x) new_s[i] = __float2bfloat16_rn(0.f);
            }
        }
    }
    __syncthreads();  // Qs and new_s visible
    if (p.kv_new != nullptr && p.inv_freq != nullptr) {
        // rotate q rows and the new k in shared memory: element j pairs with j + rotary_dim/2
        for (int r = warp; r < rows + (has_newest ? 1 : 0); r += NWARPS) {  // a row per warp at a time
            bf16* row = r < rows ? Qs + r * LD : new_s;
            for (int j = lane; j < half; j += 32) {
                const float c = cs_s[j], sn = cs_s[half + j];
                const float x1 = __bfloat162float(row[j]), x2 = __bfloat162float(row[j + half]);
                row[j] = __float2bfloat16_rn(x1 * c - x2 * sn);
                row[j + half] = __float2bfloat16_rn(x2 * c + x1 * sn);
            }
        }
        __syncthreads();
    }
    }  // (not rotate_on_load)
    if (p.kv_new != nullptr && has_newest && qg == 0) {
        // one CTA per (request, KV head) stores the new token
        const int slot = p.slots != nullptr ? p.slots[row] : -1;
        if (slot >= p.num_slots) {
            if (tid == 0) cw_report(p.status, CW_ST_SLOT_RANGE, s, slot);
        } else if (slot >= 0) {
            const size_t dst = ((size_t)slot * p.nkv + kvh) * HD;
            for (int i = tid; i < 2 * CH; i += blockDim.x)
                *reinterpret_cast<uint4*>((i < CH ? p.k_cache_w : p.v_cache_w) + dst + (i % CH) * 8) =
                    *reinterpret_cast<const uint4*>(new_s + (i < CH ? 0 : HD) + (i % CH) * 8);
        }
    }
    const int newest_tile = has_newest ? (newest - t0) / TILE : -1;
    uint32_t qa[HD / 16][4];
#pragma unroll
    for (int ks = 0; ks < HD / 16; ++ks)
        ldmatrix_x4(smem_addr(Qs + ((lane & 7) + 8 * ((lane >> 3) & 1)) * LD + ks * 16 + 8 * (lane >> 4)),
                    qa[ks][0], qa[ks][1], qa[ks][2], qa[ks][3]);

    float o_acc[HD / 8][4];
#pragma unroll
    for (int i = 0; i < HD / 8; ++i) o_acc[i][0] = o_acc[i][1] = o_acc[i][2] = o_acc[i][3] = 0.f;
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};

    for (int it = 0; it < ntiles; ++it) {
        const int buf = it % ST;
        if (TMA) {
            // (a wait that runs out is recorded and the kernel goes on: every thread keeps meeting the barriers below)
            mbar_wait(smem_addr(&full_bar[buf]), (it / ST) & 1, &give_up);
            const int pos0 = t0 + it * TILE;
            if (pos0 + TILE > t1 || pos0 < kv_begin) {
                // values of rows that are no visible key: their probabilities are zero, and zero times
                // whatever the page held there must be zero
                for (int i = tid; i < TILE * CH; i += blockDim.x) {
                    const int r = i / CH, pos = pos0 + r;
                    if (pos >= t1 || pos < kv_begin)
                        *reinterpret_cast<uint4*>(Vs + buf * TILE * LDK + kv_off(r, i % CH)) = make_uint4(0, 0, 0, 0);
                }
            }
        } else {
            cp_async_wait_upto(min(ntiles - it - 1, ST - 1));  // tile `it` has landed; later ones may fly
        }
        if (it == newest_tile) {
            const int r = newest - t0 - it * TILE;
            for (int i = tid; i < 2 * CH; i += blockDim.x)
                *reinterpret_cast<uint4*>((i < CH ? Ks : Vs) + buf * TILE * LDK + kv_off(r, i % CH)) =
                    *reinterpret_cast<const uint4*>(new_s + (i < CH ? 0 : HD) + (i % CH) * 8);
        }
        __syncthreads();
        const bf16* kt = Ks + buf * TILE * LDK;
        const bf16* vt = Vs + buf * TILE * LDK;
        const int wr = warp * 16;  // this warp's 16 rows of the tile
        const int tok0 = t0 + it * TILE + warp * 16;  // first token of this warp's 16
        if (tok0 < t1) {
            float sc[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll
            for (int ks = 0; ks < HD / 16; ++ks) {
                uint32_t b0, b1, b2, b3;
                ldmatrix_x4(smem_addr(kt + kv_off(wr + (lane & 7) + 8 * (lane >> 4), 2 * ks + ((lane >> 3) & 1))),
                            b0, b1, b2, b3);
                mma_bf16(sc[0], qa[ks], b0, b1);
                mma_bf16(sc[1], qa[ks], b2, b3);
            }
            float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
            for (int j = 0; j < 2; ++j)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int pos = tok0 + 8 * j + 2 * t + (e & 1);
                    const float v = (pos >= kv_begin && pos < t1) ? sc[j][e] * scale_log2 : -INFINITY;
                    sc[j][e] = v;
                    mx[e >> 1] = fmaxf(mx[e >> 1], v);
                }
            uint32_t pa[4];
            float alpha[2];
#pragma unroll
            for (int r = 0; r < 2; ++r) {
                mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
                mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
                const float m_new = fmaxf(m_run[r], mx[r]);
                alpha[r] = (m_run[r] == -INFINITY) ? 0.f : fast_exp2(m_run[r] - m_new);
                float sum = 0.f;
#pragma unroll
                for (int j = 0; j < 2; ++j)
#pragma unroll
                    for (int e = 0; e < 2; ++e) {
                        const float v = sc[j][2 * r + e];
                        const float pr = (m_new == -INFINITY) ? 0.f : fast_exp2(v - m_new);
                        sc[j][2 * r + e] = pr;
                        sum += pr;
                    }
                l_run[r] = l_run[r] * alpha[r] + sum;
                m_run[r] = m_new;
            }
            pa[0] = pack_bf16(sc[0][0], sc[0][1]);
            pa[1] = pack_bf16(sc[0][2], sc[0][3]);
            pa[2] = pack_bf16(sc[1][0], sc[1][1]);
            pa[3] = pack_bf16(sc[1][2], sc[1][3]);
#pragma unroll
            for (int n2 = 0; n2 < HD / 16; ++n2) {
                uint32_t v0, v1, v2, v3;
                ldmatrix_x4_trans(smem_addr(vt + kv_off(wr + (lane & 7) + 8 * ((lane >> 3) & 1), 2 * n2 + (lane >> 4))),
                                  v0, v1, v2, v3);
                float* oa = o_acc[2 * n2];
                float* ob = o_acc[2 * n2 + 1];
                oa[0] *= alpha[0]; oa[1] *= alpha[0]; oa[2] *= alpha[1]; oa[3] *= alpha[1];
                ob[0] *= alpha[0]; ob[1] *= alpha[0]; ob[2] *= alpha[1]; ob[3] *= alpha[1];
                mma_bf16(oa, pa, v0, v1);
                mma_bf16(ob, pa, v2, v3);
            }
        }
        __syncthreads();  // everyone is done with this buffer before it is refilled
        if (it + ST < ntiles) load_tile(it + ST);
    }
    if (TMA && give_up) {
        // a wait ran out: say so, and give the copies still in flight a bounded time to land before
        // the merge below writes over the tiles
        if (tid == 0) {
            cw_report(p.status, CW_ST_WAIT_TIMEOUT, blockIdx.x, -3);
            for (int k = max(0, ntiles - ST); k < ntiles; ++k) {
                const long long t_begin = clock64();
                while (!mbar_try_wait(smem_addr(&full_bar[k % ST]), (k / ST) & 1) && clock64() - t_begin < WAIT_CYCLES) {
                }
            }
        }
        __syncthreads();
    }
    // ---- merge the four warps (each saw a quarter of every tile) -----------------------------------
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 1);
        l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 2);
    }
    float* Om = (float*)Ks;  // [NWARPS][16][HD], over the K/V buffers (all reads are done)
    if (t == 0) {
        ml_s[warp][g][0] = m_run[0]; ml_s[warp][g][1] = l_run[0];
        ml_s[warp][g + 8][0] = m_run[1]; ml_s[warp][g + 8][1] = l_run[1];
    }
#pragma unroll
    for (int nt = 0; nt < HD / 8; ++nt) {
        float* base = Om + (size_t)warp * 16 * HD;
        base[g * HD + nt * 8 + 2 * t] = o_acc[nt][0];
        base[g * HD + nt * 8 + 2 * t + 1] = o_acc[nt][1];
        base[(g + 8) * HD + nt * 8 + 2 * t] = o_acc[nt][2];
        base[(g + 8) * HD + nt * 8 + 2 * t + 1] = o_acc[nt][3];
    }
    __syncthreads();
    // per query row: the warps' shares (normalised) and the split's log2-sum-exp, computed once
    if (tid < 16) {
        const int r = tid;
        float m = -INFINITY;
#pragma unroll
        for (int w = 0; w < NWARPS; ++w) m = fmaxf(m, ml_s[w][r][0]);
        float e[NWARPS], L = 0.f;
#pragma unroll
        for (int w = 0; w < NWARPS; ++w) {
            const float mw = ml_s[w][r][0];
            e[w] = (mw == -INFINITY || m == -INFINITY) ? 0.f : fast_exp2(mw - m);
            L += e[w] * ml_s[w][r][1];
        }
        const float inv = L > 0.f ? 1.f / L : 0.f;
#pragma unroll
        for (int w = 0; w < NWARPS; ++w) w_s[r][w] = e[w] * inv;
        w_s[r][NWARPS] = L > 0.f ? m + log2f(L) : -INFINITY;  // base 2
    }
    __syncthreads();
    for (int item = tid; item < rows * (HD / 4); item += blockDim.x) {  // four outputs per thread and pass
        const int r = item / (HD / 4), d = (item % (HD / 4)) * 4;
        float4 val = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int w = 0; w < NWARPS; ++w) {
            const float4 x = *reinterpret_cast<const float4*>(Om + ((size_t)w * 16 + r) * HD + d);
            const float ww = w_s[r][w];
            val.x = fmaf(ww, x.x, val.x); val.y = fmaf(ww, x.y, val.y);
            val.z = fmaf(ww, x.z, val.z); val.w = fmaf(ww, x.w, val.w);
        }
        const int h = h0 + r;
        if (active == 1) {
            uint2 o;
            o.x = pack_bf16(val.x, val.y);
            o.y = pack_bf16(val.z, val.w);
            *reinterpret_cast<uint2*>(p.out + ((size_t)row * p.nh + h) * HD + d) = o;
        } else if (CL) {
            // group `item` of four outputs belongs to the slice of split (item % active): into that CTA's
            // inbox, in this split's row of it
            const int me = sp - first_split, owner = item % active;
            const int quota = (rows * (HD / 4) + active - 1) / active;
            float4* dst = &inbox_s[me * quota + item / active];
            if (owner == me)
                *dst = val;
            else
                asm volatile("st.shared::cluster.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(peer_smem(smem_addr(dst), first_split + owner)),
                             "f"(val.x), "f"(val.y), "f"(val.z), "f"(val.w) : "memory");
        } else {
            *reinterpret_cast<float4*>(p.part_o + (((size_t)s * p.nh + h) * p.max_splits + sp) * HD + d) = val;
            if (d == 0) p.part_lse[((size_t)s * p.nh + h) * p.max_splits + sp] = w_s[r][NWARPS];
        }
    }
    if (active == 1) {
        cw_trace_end();
        return;
    }
    if (CL) {
        // ---- the splits exchange slices through the cluster and each merges its own ---------------------
        const int me = sp - first_split;
        const int items = rows * (HD / 4), quota = (items + active - 1) / active;
        for (int i = tid; i < rows * active; i += blockDim.x) {  // this split's log-sum-exps, to every split of the group
            const int k = i / rows, r = i - k * rows;
            float* dst = &lse_all[me][r];
            if (k == me)
                *dst = w_s[r][NWARPS];
            else
                asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(peer_smem(smem_addr(dst), first_split + k)), "f"(w_s[r][NWARPS]) : "memory");
        }
        __syncthreads();  // all of this CTA's pushes are issued and ordered before thread 0's arrivals
        if (tid == 0) {
            asm volatile("fence.acq_rel.cluster;" ::: "memory");
            for (int k = 0; k < active; ++k)
                if (k != me)
                    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];"
                                 ::"r"(peer_smem(smem_addr(&merge_bar), first_split + k)) : "memory");
            // the other splits' pushes have landed when all of them have arrived here
            const long long t_begin = clock64();
            uint32_t done = 0;
            while (!done) {
                asm volatile(
                    "{\n\t.reg .pred p;\n\t"
                    "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], 0;\n\t"
                    "selp.u32 %0, 1, 0, p;\n\t}"
                    : "=r"(done) : "r"(smem_addr(&merge_bar)) : "memory");
                if (!done && clock64() - t_begin > 2000000000LL) {
                    cw_report(p.status, CW_ST_WAIT_TIMEOUT, 100 + s, sp);
                    break;
                }
            }
        }
        __syncthreads();
        for (int slot = tid; slot < quota; slot += blockDim.x) {
            const int item = slot * active + me;
            if (item >= items) continue;
            const int r = item / (HD / 4), d = (item % (HD / 4)) * 4;
            float m = -INFINITY, W = 0.f;
            float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 1
            for (int k = 0; k < active; ++k) m = fmaxf(m, lse_all[k][r]);
#pragma unroll 4
            for (int k = 0; k < active; ++k) {  // sources in split order
                const float lk = lse_all[k][r];
                const float4 x = inbox_s[k * quota + slot];
                const float w = (lk == -INFINITY) ? 0.f : fast_exp2(lk - m);
                W += w;
                acc.x = fmaf(w, x.x, acc.x); acc.y = fmaf(w, x.y, acc.y);
                acc.z = fmaf(w, x.z, acc.z); acc.w = fmaf(w, x.w, acc.w);
            }
            const float inv = W > 0.f ? 1.f / W : 0.f;
            uint2 o;
            o.x = pack_bf16(acc.x * inv, acc.y * inv);
            o.y = pack_bf16(acc.z * inv, acc.w * inv);
            *reinterpret_cast<uint2*>(p.out + ((size_t)row * p.nh + h0 + r) * HD + d) = o;
        }
        cw_trace_end();
        return;
    }
    // ---- the CTA that finishes last merges the splits, in split order ------------------------------
    // Up to 36 splits meet at the group's counter and the last one merges them all (further down).
    // More splits (a long context of few requests) meet in two levels, so that the merge is not one
    // CTA's walk over hundreds of partials: twelve consecutive splits share a counter of their own, the
    // last of them merges the twelve into the first one's place in the workspace (a normalised partial
    // with its log-sum-exp, like those it read), and the last of these mergers to arrive at the group's
    // counter merges their results.  The order of the additions depends on the number of splits only,
    // never on who arrives last.  (TREE: a variant of its own, launched for the few requests with long
    // contexts that can make so many splits; the kernel of the usual step does not hold this code, since a
    // decode CTA's time is made of the instructions it has to fetch.)
    constexpr int Q4 = HD / 4;
    constexpr int KC = 12;
    if (TREE && active > 3 * KC) {
        const size_t group = ((size_t)s * p.nkv + kvh) * p.qgroups + qg;
        const int sub = (sp - first_split) / KC, max_subs = (p.max_splits + KC - 1) / KC;
        // the partials this CTA merges if it is the last to arrive: first, first + stride, ..
        int first = sub * KC, count = min(KC, active - first), stride = 1;
        int* counter = p.counters + (size_t)gridDim.x * gridDim.y + group * max_subs + sub;
        bool final = false;
#pragma unroll 1
        for (;;) {
            __syncthreads();
            if (tid == 0) {
                int prev;
                asm volatile("atom.add.acq_rel.gpu.global.s32 %0, [%1], 1;" : "=r"(prev) : "l"(counter) : "memory");
                last_flag = (prev == count - 1);
                if (last_flag) *counter = 0;
            }
            __syncthreads();
            if (!last_flag) break;
            for (int item = tid; item < rows * Q4; item += blockDim.x) {
                const int r = item / Q4, d = (item % Q4) * 4;
                float* lp = p.part_lse + ((size_t)s * p.nh + h0 + r) * p.max_splits + first_split + first;
                float4* po = reinterpret_cast<float4*>(
                    p.part_o + (((size_t)s * p.nh + h0 + r) * p.max_splits + first_split + first) * HD + d);
                float m = -INFINITY, W = 0.f;
                float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 1
                for (int k0 = 0; k0 < count; k0 += KC) {
                    float l[KC];
                    float4 v[KC];
#pragma unroll
                    for (int k = 0; k < KC; ++k) {
                        l[k] = k0 + k < count ? __ldcg(lp + (k0 + k) * stride) : -INFINITY;
                        v[k] = k0 + k < count ? __ldcg(po + (size_t)(k0 + k) * stride * Q4) : make_float4(0.f, 0.f, 0.f, 0.f);
                    }
                    float m_new = m;
#pragma unroll
                    for (int k = 0; k < KC; ++k) m_new = fmaxf(m_new, l[k]);
                    if (k0 > 0) {
                        const float keep = (m == -INFINITY) ? 0.f : fast_exp2(m - m_new);
                        W *= keep;
                        acc.x *= keep; acc.y *= keep; acc.z *= keep; acc.w *= keep;
                    }
                    m = m_new;
#pragma unroll
                    for (int k = 0; k < KC; ++k) {
                        const float w = (l[k] == -INFINITY) ? 0.f : fast_exp2(l[k] - m);
                        W += w;
                        acc.x = fmaf(w, v[k].x, acc.x); acc.y = fmaf(w, v[k].y, acc.y);
                        acc.z = fmaf(w, v[k].z, acc.z); acc.w = fmaf(w, v[k].w, acc.w);
                    }
                }
                const float inv = W > 0.f ? 1.f / W : 0.f;
                if (final) {
                    uint2 o;
                    o.x = pack_bf16(acc.x * inv, acc.y * inv);
                    o.y = pack_bf16(acc.z * inv, acc.w * inv);
                    *reinterpret_cast<uint2*>(p.out + ((size_t)row * p.nh + h0 + r) * HD + d) = o;
                } else {
                    // over the first of the twelve: this thread alone reads and writes these four outputs
                    *po = make_float4(acc.x * inv, acc.y * inv, acc.z * inv, acc.w * inv);
                    if (d == 0) w_s[r][0] = W > 0.f ? m + log2f(W) : -INFINITY;
                }
            }
            if (final) break;
            // the merged log-sum-exps go over the first split's once every thread has read those
            __syncthreads();
            if (tid < rows) p.part_lse[((size_t)s * p.nh + h0 + tid) * p.max_splits + first_split + first] = w_s[tid][0];
            count = (active + KC - 1) / KC;
            first = 0;
            stride = KC;
            counter = p.counters + group;
            final = true;
        }
        cw_trace_end();
        return;
    }
    // Release / acquire through the counter: the barrier orders every thread's partial stores before
    // thread 0's release at GPU scope, and the last CTA's acquire, followed by its barrier, orders its
    // threads' loads after all groups' stores.  (One scoped atomic instead of a fence in every thread.)
    __syncthreads();
    if (tid == 0) {
        int* counter = p.counters + ((size_t)s * p.nkv + kvh) * p.qgroups + qg;
        int prev;
        asm volatile("atom.add.acq_rel.gpu.global.s32 %0, [%1], 1;" : "=r"(prev) : "l"(counter) : "memory");
        last_flag = (prev == active - 1);
        if (last_flag) *counter = 0;
    }
    __syncthreads();
    if (!last_flag) {
        cw_trace_end();
        return;
    }
    // Every thread merges groups of four outputs: weights w_k = 2^(lse_k - max) and the weighted sum of
    // the splits' partials, divided by the sum of the weights at the end, splits in order.  The splits
    // are taken twelve at a time, and all loads of a round (the row's log-sum-exps and the partials) are
    // issued before any is used: one trip to the L2 per round.  Between rounds the sum so far is
    // rescaled to the new maximum, as in the online softmax.
    for (int item = tid; item < rows * Q4; item += blockDim.x) {
        const int r = item / Q4, d = (item % Q4) * 4;
        const float* lp = p.part_lse + ((size_t)s * p.nh + h0 + r) * p.max_splits + first_split;
        const float4* po = reinterpret_cast<const float4*>(
            p.part_o + (((size_t)s * p.nh + h0 + r) * p.max_splits + first_split) * HD + d);
        float m = -INFINITY, W = 0.f;
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 1
        for (int k0 = 0; k0 < active; k0 += KC) {
            float l[KC];
            float4 v[KC];
#pragma unroll
            for (int k = 0; k < KC; ++k) {
                l[k] = k0 + k < active ? __ldcg(lp + k0 + k) : -INFINITY;
                v[k] = k0 + k < active ? __ldcg(po + (size_t)(k0 + k) * Q4) : make_float4(0.f, 0.f, 0.f, 0.f);
            }
            float m_new = m;
#pragma unroll
            for (int k = 0; k < KC; ++k) m_new = fmaxf(m_new, l[k]);
            if (k0 > 0) {
                const float keep = (m == -INFINITY) ? 0.f : fast_exp2(m - m_new);
                W *= keep;
                acc.x *= keep; acc.y *= keep; acc.z *= keep; acc.w *= keep;
            }
            m = m_new;
#pragma unroll
            for (int k = 0; k < KC; ++k) {
                const float w = (l[k] == -INFINITY) ? 0.f : fast_exp2(l[k] - m);
                W += w;
                acc.x = fmaf(w, v[k].x, acc.x); acc.y = fmaf(w, v[k].y, acc.y);
                acc.z = fmaf(w, v[k].z, acc.z); acc.w = fmaf(w, v[k].w, acc.w);
            }
        }
        const float inv = W > 0.f ? 1.f / W : 0.f;
        uint2 o;
        o.x = pack_bf16(acc.x * inv, acc.y * inv);
        o.y = pack_bf16(acc.z * inv, acc.w * inv);
        *reinterpret_cast<uint2*>(p.out + ((size_t)row * p.nh + h0 + r) * HD + d) = o;
    }
    cw_trace_end();
}

static CUtensorMap g_no_map;  // what the variants without TMA are given (one per translation unit)

template <int HD, int ST, int LAYOUT, bool CL, bool TREE = false>
static int launch_decode_cl(const DecodeParams& p, int S, int splits, cudaStream_t stream, const CUtensorMap& mk = g_no_map,
                            const CUtensorMap& mv = g_no_map) {
    constexpr int LD = HD + 8;
    constexpr int LDK = (LAYOUT != KV_PADDED && HD % 64 == 0) ? HD : HD + 8;
    const int SMEM = (16 * LD + 2 * ST * TILE * LDK) * 2 + p.max_split_pages * 4;
    constexpr int MERGE = NWARPS * 16 * HD * 4;
    static_assert(MERGE <= 2 * ST * TILE * LDK * 2, "the merge buffer must fit over the K and V buffers");
    static int configured = 0;
    if (SMEM > configured) {
        if (SMEM > 48 * 1024 &&
            cudaFuncSetAttribute(attn_decode_kernel<HD, ST, LAYOUT, CL, TREE>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM) != cudaSuccess)
            return (int)cudaGetLastError();
        if (CL && cudaFuncSetAttribute(attn_decode_kernel<HD, ST, LAYOUT, CL, TREE>, cudaFuncAttributeNonPortableClusterSizeAllowed, 1) != cudaSuccess)
            return (int)cudaGetLastError();
        configured = SMEM;
    }
    dim3 grid(p.nkv * p.qgroups, S, splits);
    return cw_launch(attn_decode_kernel<HD, ST, LAYOUT, CL, TREE>, grid, dim3(NWARPS * 32), SMEM, stream, CL ? (unsigned)splits : 1u, mk, mv, p);
}

template <int HD, int ST, int LAYOUT>
static int launch_decode_st(const DecodeParams& p, int S, int splits, cudaStream_t stream) {
    // (the cluster form for head sizes up to 128: the larger ones have no room for its inbox beside their tiles)
    if (HD <= 128 && p.cluster > 1) return launch_decode_cl<HD, ST, LAYOUT, (HD <= 128)>(p, S, splits, stream);
    if (ST == 2 && p.tree) return launch_decode_cl<HD, ST, LAYOUT, false, (ST == 2)>(p, S, splits, stream);
    return launch_decode_cl<HD, ST, LAYOUT, false>(p, S, splits, stream);
}

// The cache as [64 elements][slot][64-element block][kv head]: a box is one page of one head with all its
// blocks, which land one after the other ([block][token][128 bytes], 128-byte swizzle).
static int page_map(CUtensorMap* map, const void* cache, int num_pages, int page_size, int nkv, int hd) {
    const cuuint64_t dims[4] = {64, (cuuint64_t)num_pages * page_size, (cuuint64_t)(hd / 64), (cuuint64_t)nkv};
    const cuuint64_t strides[3] = {(cuuint64_t)nkv * hd * 2, 128, (cuuint64_t)hd * 2};
    const cuuint32_t box[4] = {64, (cuuint32_t)page_size, (cuuint32_t)(hd / 64), 1};
    const cuuint32_t elem[4] = {1, 1, 1, 1};
    return g_encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(cache), dims, strides, box, elem,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS ? 0 : -1;
}

template <int HD, int ST>
static int launch_decode_tma(const DecodeParams& p, int S, int splits, cudaStream_t stream) {
    CUtensorMap mk, mv;
    if (load_encode() != 0) return CW_ERR_UNSUPPORTED;  // (the encoder's address is kept per translation unit)
    if (page_map(&mk, p.k_cache, p.num_pages, p.page_size, p.nkv, HD) != 0 || page_map(&mv, p.v_cache, p.num_pages, p.page_size, p.nkv, HD) != 0)
        return CW_ERR_UNSUPPORTED;
    if (ST == 2 && p.tree) return launch_decode_cl<HD, ST, KV_TMA, false, (ST == 2)>(p, S, splits, stream, mk, mv);
    return launch_decode_cl<HD, ST, KV_TMA, false>(p, S, splits, stream, mk, mv);
}

template <int HD>
static int launch_decode(const DecodeParams& p, int S, int splits, cudaStream_t stream) {
    // Four tiles in flight per CTA (one CTA per SM) suit steps with few CTAs, where latency is
    // everything; with many CTAs two tiles in flight leave room for two or three CTAs per SM, and
    // the warps of the others cover each CTA's stalls.
    if (HD % 64 == 0 && p.tma) {
        if (HD <= 128 && p.stages != 2) return launch_decode_tma<(HD % 64 == 0 ? HD : 64), (HD <= 128 ? 4 : 2)>(p, S, splits, stream);
        return launch_decode_tma<(HD % 64 == 0 ? HD : 64), 2>(p, S, splits, stream);
    }
    if (HD <= 128 && p.stages != 2) return launch_decode_st<HD, (HD <= 128 ? 4 : 2), KV_PADDED>(p, S, splits, stream);
    if (HD % 64 == 0 && p.swizzle) return launch_decode_st<HD, 2, (HD % 64 == 0 ? KV_SWIZZLED : KV_PADDED)>(p, S, splits, stream);
    return launch_decode_st<HD, 2, KV_PADDED>(p, S, splits, stream);
}


// The head sizes are compiled in three translation units (a third of the build's time each): up to 64
// beside the entry points, 80 to 128 in attention_decode_mid.cu, the larger ones in attention_decode_large.cu.
int cw_launch_decode_mid(int hd, const DecodeParams& p, int S, int splits, cudaStream_t stream);
int cw_launch_decode_large(int hd, const DecodeParams& p, int S, int splits, cudaStream_t stream);
