// The matrix product for prompt portions on CTA pairs (tcgen05 cta_group::2).
//
// Two CTAs of a cluster, on neighbouring SMs, share one tile of 256 output features x bn tokens:
// each loads its own 128 rows of W and only half of the token tile, and the leader's one thread
// issues MMAs of M = 256 that run on both SMs' tensor cores and read the token tile from both
// shared memories.  Against two independent 128 x bn tiles that halves the token-operand traffic
// per SM (TMA writes and tensor-core reads of shared memory), which is what bounds the single-CTA
// kernel.  Each CTA keeps the accumulator of its own 128 features in its own tensor memory (two
// buffers: the epilogue of one tile overlaps the MMAs of the next) and stores it itself.
//
// Barriers: `full[s]` lives in the leader and counts one arrive.expect_tx per CTA plus the bytes
// of both CTAs' copies (the peer's copies signal it through the cluster's shared-memory window);
// `empty[s]` and `acc_full[b]` are signalled in both CTAs at once by a multicast tcgen05.commit;
// `acc_empty[b]` lives in the leader and counts one arrival per CTA's epilogue.  Every wait is
// bounded; a CTA that gives up records CW_ST_WAIT_TIMEOUT, and both CTAs meet at the cluster
// barrier before tensor memory is freed.
//
// Few tiles and a long inner dimension (a few hundred tokens against K = 8960): a pair streams its
// weight rows at the rate its six stages in flight allow (about 3 k-blocks per microsecond), so
// with fewer tiles than pairs the product's time is K's, whatever the tile's width.  The products
// that add into the residual are then split over K (p.splits > 1): a unit of work is (tile, split),
// every split adds its partial tile into the residual with the same TMA reduce-add, and the splits
// of a tile add in split order: split k waits, before its first store, until split k - 1 has
// published (p.split_flags[tile] == k) that its stores are complete.  Units are handed out in the
// order (tile, split) to pairs that all run at once and take their units in ascending order, so the
// unit waited for is always running or done.
#pragma once
#include "tc_common.cuh"

#define PAIR_THREADS 192
#define PAIR_CHUNK 16            // tokens per epilogue store
#define PAIR_MAX_SMEM (227 * 1024)

// SWIGLU: two weight matrices (gate and up) against the same token tile, two accumulators per tile, and
// silu(gate) * up in the epilogue; token tiles are then at most 128 wide (tensor memory holds two
// buffers of two accumulators).
template <bool SWIGLU>
struct PairCfgT {
    static constexpr int BN_MAX = SWIGLU ? 128 : 256;            // BM = 128 and BK = 64 as in the single-CTA kernels
    static constexpr int ACC_STRIDE = 256;                       // tensor-memory columns per buffer (SWIGLU: gate at 0, up at 128)
    static constexpr int A_BYTES = BM * BK * 2;                  // this CTA's 128 rows of W (of each W)
    static constexpr int B_BYTES = (BN_MAX / 2) * BK * 2;        // its half of the token tile
    static constexpr int STAGE_BYTES = (SWIGLU ? 2 : 1) * A_BYTES + B_BYTES;
    static constexpr int OUT_BYTES = 2 * PAIR_CHUNK * BM * 4;    // two staging buffers of [16 tokens][128 features]
    static constexpr int STAGES = (PAIR_MAX_SMEM - 2048 - OUT_BYTES) / STAGE_BYTES;
    static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + OUT_BYTES + 1024 + 1024;
    static constexpr int TMEM_COLS = 512;                        // two buffers of up to 256 columns
    static_assert(STAGES >= 4, "too few operand stages");
};
using PairCfg = PairCfgT<false>;

__device__ __forceinline__ void tmem_alloc_pair(uint32_t result_slot, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(result_slot), "r"(cols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void umma_bf16_pair(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                               uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// Arrives, when the MMAs issued so far are complete, on the barrier at this offset in both CTAs.
__device__ __forceinline__ void umma_commit_pair(uint32_t bar) {
    asm volatile(
        "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
        ::"r"(bar), "h"((uint16_t)3)
        : "memory");
}
// A tile copy whose completion bytes go to a barrier that may lie in the other CTA of the pair.
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t cluster_bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst), "l"(map), "r"(cluster_bar), "r"(x), "r"(y)
        : "memory");
}
__device__ __forceinline__ void mbar_expect_tx_cluster(uint32_t cluster_bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cluster.b64 _, [%0], %1;" ::"r"(cluster_bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_bar) {
    asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_bar) : "memory");
}

// Tiles: 256 features x p.bn tokens per pair; p.bn is a multiple of 16 (each CTA holds p.bn / 2 token
// rows, whole swizzle atoms of 8).  map_x's box is p.bn / 2 rows, map_c's box [16 tokens][128 features].
template <bool SWIGLU>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(PAIR_THREADS, 1)
gemm_tc_pair_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_w2,
                    const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_c, const GemmParams p) {
    using C = PairCfgT<SWIGLU>;
    constexpr int B_OFF = (SWIGLU ? 2 : 1) * C::A_BYTES;  // the token rows' place in a stage
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t* out_s = smem + C::STAGES * C::STAGE_BYTES;
    uint64_t* bars = (uint64_t*)(out_s + C::OUT_BYTES);
    // bars: full[S], empty[S], acc_full[2], acc_empty[2]
    uint32_t* tmem_slot = (uint32_t*)(bars + 2 * C::STAGES + 4);
    volatile int* give_up = (volatile int*)(tmem_slot + 1);

    // Only the activations come from the preceding kernel, and only the producer threads read them
    // (everything else follows from their copies): they alone wait for it, after the set-up and after
    // the weight tiles of the first stages have gone out.
    pdl_launch_dependents();
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t rank = cluster_rank();  // 0: the leader, which issues the MMAs
    const uint32_t full0 = smem_u32(bars), empty0 = smem_u32(bars + C::STAGES);
    const uint32_t accf0 = smem_u32(bars + 2 * C::STAGES), acce0 = smem_u32(bars + 2 * C::STAGES + 2);
    const int bn = p.bn, half_bn = bn >> 1;
    const int m_tiles = (p.N + 2 * BM - 1) / (2 * BM), n_tiles = (p.T + bn - 1) / bn;
    const int splits = p.splits, nkb = p.kb_per_split;  // splits * nkb == p.num_kb
    const int tiles = m_tiles * n_tiles * splits;       // units of work: unit u is split u % splits of tile u / splits
    const int pair = blockIdx.x >> 1, pairs = gridDim.x >> 1;

    if (tid == 0) {
        for (int s = 0; s < C::STAGES; ++s) {
            mbar_init(full0 + 8 * s, 2);   // one arrive.expect_tx per CTA (used in the leader only)
            mbar_init(empty0 + 8 * s, 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(accf0 + 8 * b, 1);
            mbar_init(acce0 + 8 * b, 2);   // one arrival per CTA's epilogue (used in the leader only)
        }
        *give_up = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) tmem_alloc_pair(smem_u32(tmem_slot), C::TMEM_COLS);
    tc_fence_before();
    cluster_sync();  // both CTAs' barriers are initialised before either signals the other's
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0 && lane == 0) {
        // ---- TMA producer (both CTAs): own rows of W, own half of the token tile ------------------------
        const uint32_t stage_tx = B_OFF + half_bn * BK * 2;
        const int my_tiles = pair < tiles ? (tiles - pair + pairs - 1) / pairs : 0;
        const int total = my_tiles * nkb;  // k-blocks of all this pair's units, in order
        const int early = min(total, C::STAGES);
        bool ok = true;
        int i = 0;
        // the first stages: weight tiles before the wait, their activation tiles after it
        for (int phase = 0; phase < 2; ++phase) {
            if (phase == 1) pdl_wait();
            for (i = 0; i < early; ++i) {
                const int ts = i / nkb, unit = pair + ts * pairs, tile = unit / splits;
                const int kb = (unit - tile * splits) * nkb + (i - ts * nkb);  // k-block within K
                const int m0 = (tile % m_tiles) * 2 * BM + (int)rank * BM;
                const int n0 = (tile / m_tiles) * bn + (int)rank * half_bn;
                const uint32_t a_dst = smem_u32(smem + i * C::STAGE_BYTES);
                const uint32_t bar = dsmem_addr(full0 + 8 * i, 0);  // the leader's barrier
                if (phase == 0) {
                    mbar_expect_tx_cluster(bar, stage_tx);
                    tma_load_2d_pair(a_dst, &map_w, kb * BK, m0, bar);
                    if (SWIGLU) tma_load_2d_pair(a_dst + C::A_BYTES, &map_w2, kb * BK, m0, bar);
                } else {
                    tma_load_2d_pair(a_dst + B_OFF, &map_x, kb * BK, n0, bar);
                }
            }
        }
        // the rest runs ahead over tiles, bounded by the ring only
        int kb = early % nkb;
        for (int unit = pair + (early / nkb) * pairs; unit < tiles && ok; unit += pairs, kb = 0) {
            const int tile = unit / splits, kb0 = (unit - tile * splits) * nkb;
            const int m0 = (tile % m_tiles) * 2 * BM + (int)rank * BM;
            const int n0 = (tile / m_tiles) * bn + (int)rank * half_bn;
            for (; kb < nkb; ++kb, ++i) {
                const int s = i % C::STAGES;
                ok = mbar_wait(empty0 + 8 * s, ((i / C::STAGES) & 1) ^ 1, give_up);
                if (!ok) break;
                const uint32_t a_dst = smem_u32(smem + s * C::STAGE_BYTES);
                const uint32_t bar = dsmem_addr(full0 + 8 * s, 0);  // the leader's barrier
                mbar_expect_tx_cluster(bar, stage_tx);
                tma_load_2d_pair(a_dst, &map_w, (kb0 + kb) * BK, m0, bar);
                if (SWIGLU) tma_load_2d_pair(a_dst + C::A_BYTES, &map_w2, (kb0 + kb) * BK, m0, bar);
                tma_load_2d_pair(a_dst + B_OFF, &map_x, (kb0 + kb) * BK, n0, bar);
            }
        }
        if (*give_up) {
            // copies may still be in flight into this CTA's shared memory, and their barrier lies in the
            // leader: let them land before the CTA goes on to the final barrier and leaves
            const long long t0 = clock64();
            while (clock64() - t0 < 2000000LL) {
            }
        }
    } else if (warp == 1 && lane == 0 && rank == 0) {
        // ---- MMA issuer (leader only): tile `it` accumulates into TMEM buffer it & 1 of both CTAs ---------
        pdl_wait();  // (parked here a thread polls no barrier)
        const uint32_t idesc = instr_desc(2 * BM, bn);
        int i = 0, it = 0;
        bool ok = true;
        for (int tile = pair; tile < tiles && ok; tile += pairs, ++it) {
            const int buf = it & 1;
            ok = mbar_wait(acce0 + 8 * buf, ((it >> 1) & 1) ^ 1, give_up);  // both epilogues have drained it
            if (!ok) break;
            tc_fence_after();
            const uint32_t acc = tmem_base + buf * C::ACC_STRIDE;
            for (int kb = 0; kb < nkb; ++kb, ++i) {
                const int s = i % C::STAGES;
                ok = mbar_wait(full0 + 8 * s, (i / C::STAGES) & 1, give_up);
                if (!ok) break;
                tc_fence_after();
                const uint32_t a_addr = smem_u32(smem + s * C::STAGE_BYTES);
                const uint64_t adesc = smem_desc_sw128(a_addr);
                const uint64_t bdesc = smem_desc_sw128(a_addr + B_OFF);
#pragma unroll
                for (int k = 0; k < BK / 16; ++k)
                    umma_bf16_pair(acc, adesc + 2 * k, bdesc + 2 * k, idesc, (kb > 0 || k > 0) ? 1u : 0u);
                if (SWIGLU) {
                    const uint64_t udesc = smem_desc_sw128(a_addr + C::A_BYTES);
#pragma unroll
                    for (int k = 0; k < BK / 16; ++k)
                        umma_bf16_pair(acc + C::ACC_STRIDE / 2, udesc + 2 * k, bdesc + 2 * k, idesc, (kb > 0 || k > 0) ? 1u : 0u);
                }
                umma_commit_pair(empty0 + 8 * s);  // the stage is free in both CTAs
            }
            if (ok) umma_commit_pair(accf0 + 8 * buf);
        }
    } else if (warp >= 2) {
        // ---- epilogue warps (both CTAs): warp w reads TMEM lanes 32 (w % 4) .. +31 of its own CTA --------
        pdl_wait();
        const int quarter = warp & 3;
        const int row = quarter * 32 + lane;
        const int etid = tid - 64;
        const bool wide = !SWIGLU && p.epilogue != 0;
        const uint32_t acce_leader = dsmem_addr(acce0, 0);
        int it = 0, chunk_no = 0;
        bool ok = true;
        for (int unit = pair; unit < tiles && ok; unit += pairs, ++it) {
            const int buf = it & 1;
            const int tile = unit / splits, ks = unit - tile * splits;
            const int m0 = (tile % m_tiles) * 2 * BM + (int)rank * BM;
            const int n0 = (tile / m_tiles) * bn;
            const int f = m0 + row;
            // (a split's adds come after those of the split before it; splits that are kept apart, epilogue
            // 3, store into slabs of their own and wait for nobody)
            const bool apart = p.epilogue == 3;
            bool my_turn = ks == 0 || apart;
            const int y0 = (apart ? ks * p.part_rows : 0) + n0;  // the tile's first row in C
            ok = mbar_wait(accf0 + 8 * buf, (it >> 1) & 1, give_up);
            {
                // one decision for all 128 threads: they meet at named barriers below
                uint32_t all_ok;
                asm volatile(
                    "{ .reg .pred p, q; setp.ne.u32 q, %1, 0; bar.red.and.pred p, 3, 128, q; selp.u32 %0, 1, 0, p; }"
                    : "=r"(all_ok)
                    : "r"((uint32_t)ok)
                    : "memory");
                ok = all_ok != 0;
            }
            if (!ok) break;
            tc_fence_after();
            const uint32_t taddr = tmem_base + buf * C::ACC_STRIDE + ((uint32_t)(quarter * 32) << 16);
            const float bias = (p.bias != nullptr && f < p.N && ks == 0) ? p.bias[f] : 0.f;
            // Only chunks that hold tokens are read out and stored, and every chunk that runs commits exactly
            // one bulk group (an empty one when this CTA's features lie beyond N), so that `wait_group.read 1`
            // below means what it says: the store that read this staging buffer two chunks ago is done with it.
            const int c_end = min(bn, p.T - n0);
            for (int c = 0; c < c_end; c += PAIR_CHUNK, ++chunk_no) {
                float g[16];
                tmem_ld16(taddr + c, g);
                if (SWIGLU) {
                    float u[16];
                    tmem_ld16(taddr + C::ACC_STRIDE / 2 + c, u);
#pragma unroll
                    for (int j = 0; j < 16; ++j) g[j] = __fdividef(g[j], 1.0f + __expf(-g[j])) * u[j];
                }
                if (c + PAIR_CHUNK >= c_end) {
                    // the accumulator has been read out: hand the buffer back to the leader's MMA thread
                    tc_fence_before();
                    asm volatile("bar.sync 1, 128;" ::: "memory");
                    if (etid == 0) mbar_arrive_cluster(acce_leader + 8 * buf);
                }
                float* st32 = (float*)(out_s + (chunk_no & 1) * (C::OUT_BYTES / 2));
                // the store that used this staging buffer two chunks ago must have read it
                if (etid == 0) asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
                asm volatile("bar.sync 2, 128;" ::: "memory");
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                    const float v = g[j] + bias;
                    if (wide)
                        st32[j * BM + row] = v;
                    else
                        ((bf16*)st32)[j * BM + row] = __float2bfloat16_rn(v);
                }
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                asm volatile("bar.sync 1, 128;" ::: "memory");
                if (etid == 0) {
                    if (!my_turn) {
                        // both CTAs of the pair hold the same tile: each waits for itself
                        const long long t0 = clock64();
                        int seen;
                        do {
                            asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(seen) : "l"(p.split_flags + 2 * tile + rank) : "memory");
                        } while (seen != ks && clock64() - t0 < WAIT_CYCLES);
                        if (seen != ks) *give_up = 1;
                        my_turn = true;
                    }
                    if (m0 < p.N) {
                        if (p.epilogue == 1)
                            asm volatile("cp.reduce.async.bulk.tensor.2d.global.shared::cta.add.bulk_group [%0, {%2, %3}], [%1];"
                                         ::"l"(&map_c), "r"(smem_u32(st32)), "r"(m0), "r"(y0 + c) : "memory");
                        else
                            asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
                                         ::"l"(&map_c), "r"(smem_u32(st32)), "r"(m0), "r"(y0 + c) : "memory");
                    }
                    asm volatile("cp.async.bulk.commit_group;" ::: "memory");
                }
            }
            if (splits > 1 && !apart && etid == 0) {
                // this split's adds are complete: the next split of the tile may add (the last one leaves
                // the flag at zero for the next launch)
                asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
                const int next = ks + 1 == splits ? 0 : ks + 1;
                asm volatile("st.release.gpu.global.s32 [%0], %1;" ::"l"(p.split_flags + 2 * tile + rank), "r"(next) : "memory");
            }
        }
        if (etid == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");  // all stores done before exit
    }
    __syncwarp();
    if (*give_up && tid == 0) cw_report(p.status, CW_ST_WAIT_TIMEOUT, blockIdx.x, -2);
    // Neither CTA leaves, or frees tensor memory, while the other may still signal its barriers or
    // while MMAs that read its shared memory may be in flight.
    tc_fence_before();
    cluster_sync();
    if (warp == 1) tmem_dealloc_pair(tmem_base, C::TMEM_COLS);
}
