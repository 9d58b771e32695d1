// bfloat16 matrix products on the 5th-generation tensor cores (tcgen05), operands staged by TMA,
// accumulators in tensor memory.
//
//   C[T, N] = X[T, K] * W[N, K]^T (+ bias[N])       W in nn.Linear layout, X the activations
//   (reference: clockwork/engine/model.py:58-60, 74-77, 88-90, 128, 216; SwiGLU :62-63)
//
// The weights ride the MMA's M dimension: one CTA owns 128 rows of W (128 output features) and a
// tile of BN tokens, so the instruction is M=128 x N=BN x K=16 with both operands K-major in
// shared memory (128-byte swizzle) and D[feature, token] in TMEM.  Three kernels:
//
//   gemm_tc_kernel             BN = 16..256, one tile per CTA: decode and short portions.  When the
//                              grid would leave SMs idle the K dimension is split over blockIdx.z and
//                              the CTAs of one tile are launched as a thread-block cluster: each
//                              pushes the columns of its partial accumulator into the shared memory
//                              of the column's owner (st.async into distributed shared memory, counted
//                              by a transaction barrier of the owner), and every owner adds what it
//                              received, in rank order, and finishes its slice of columns.  No global
//                              scratch, no atomics, no cluster-wide barrier after the main loop, and
//                              the result does not depend on which CTA finished first.
//   gemm_tc_persistent_kernel  prompt portions (more than 256 tokens): one CTA per SM walks tiles with
//                              two TMEM accumulators (the epilogue of a tile overlaps the next one's MMAs);
//                              also few tokens against three rounds of weight tiles or more (the logits)
//   gemm_tc_pair_kernel        the same on CTA pairs (cta_group::2), in gemm_tc_pair.cuh
//
// Warp roles of gemm_tc_kernel (128 threads): warp 0 lane 0 issues TMA loads, warp 1 lane 0 issues the
// MMAs, warp 2 allocates and frees TMEM; all four warps run the epilogue (warp w reads TMEM lanes
// 32w..32w+31).  Epilogues: 0 store bf16; 1 add into the float32 residual; 2 store float32; SWIGLU
// computes silu(X Wg^T) * (X Wu^T) from two accumulators; an RMSNorm can be split over the two products
// around it (GemmParams).  A decode CTA runs its epilogue exactly once, so the epilogue is written for
// a small *executed* instruction footprint (forms for 4, 8 and 16 columns, one loop per epilogue kind).
//
// Every wait on an mbarrier is bounded: when it runs out the kernel records CW_ST_WAIT_TIMEOUT in
// the status words, the producer waits (bounded again) for the copies it has in flight, TMEM is
// freed and the kernel returns.
#include "tc_common.cuh"
#include <type_traits>

#define BM 128
#define BK 64
#define THREADS 128
#define MAX_SPLITS 8  // the portable cluster size

struct GemmParams {
    int T, N, K;          // tokens, output features, inner size
    int ldc;              // row stride of C in elements
    int epilogue;         // 0 bf16 store, 1 float32 add, 2 float32 store (ignored for SWIGLU);
                          // 3 (CTA-pair kernel): float32 store of split ks at rows ks * part_rows .. of C
    int part_rows;        // epilogue 3: rows per split in C (the token count rounded up to the store's 16 rows)
    int num_kb;           // ceil(K / 64)
    int kb_per_split;     // k-blocks per blockIdx.z
    int splits;
    int bn;               // persistent kernel: token-tile width chosen at run time (multiple of 16)
    int tma_store;        // 1: unsplit tiles leave through shared memory and one TMA store / reduce-add
    const float* bias;    // [N] or null
    void* C;
    int* status;
    // An RMSNorm between two products, split over them (gemm_tc_kernel only, token tiles up to 128).
    // The product before the norm (epilogue 1, the new residual C in hand) also writes
    // emit_x[t, f] = bf16(C[t, f] * emit_g[f]) and, per 128-feature tile, emit_part[t, tile] = the sum of
    // C[t, f]^2 over the tile's features.  The product after the norm takes emit_x as X and finishes
    // the norm in its epilogue: acc * rsqrt(sum(scale_part[t, :]) / scale_dim + scale_eps) (+ bias).
    const float* scale_part;  // [T, scale_parts] or null
    int scale_parts;
    float scale_eps;
    int scale_dim;
    const float* emit_g;      // [N] or null
    bf16* emit_x;             // [T, N]
    float* emit_part;         // [T, gridDim.x]
    int* split_flags;         // CTA-pair kernel with splits > 1: two words per tile, zero between launches
};

#include "gemm_tc_pair.cuh"

template <int BN, bool SWIGLU>
struct Cfg {
    static constexpr int A_BYTES = BM * BK * 2;                     // 16 KB
    static constexpr int B_BYTES = BN * BK * 2;
    static constexpr int STAGE_BYTES = A_BYTES * (SWIGLU ? 2 : 1) + B_BYTES;
    static constexpr int ACC_COLS = BN * (SWIGLU ? 2 : 1);
    // Split-K inbox: the partial columns that the other CTAs of the cluster push into this CTA.  It
    // must not overlap the operand stages (a peer may push while this CTA's MMAs still read them).
    // Tiles too large to leave room for it are never split.
    static constexpr bool CAN_SPLIT = BN <= 64 || (BN == 128 && !SWIGLU);
    static constexpr int INBOX_BYTES = CAN_SPLIT ? (BN + MAX_SPLITS) * (SWIGLU ? 2 : 1) * BM * 4 : 0;
    // as many stages as fit (at most 8): a decode CTA is alone on its SM and keeps that many weight
    // tiles in flight from HBM
    // Small token tiles without SwiGLU (the decode products around attention) leave room for a CTA of
    // the decode attention kernel beside them, so that its prologue runs while this kernel finishes.
    static constexpr int BUDGET = (BN <= 64 && !SWIGLU) ? 140 * 1024 : 200 * 1024;
    static constexpr int MAX_STAGES = (BUDGET - INBOX_BYTES) / STAGE_BYTES;
    static constexpr int STAGES = MAX_STAGES > 8 ? 8 : MAX_STAGES;
    static constexpr int TMEM_COLS = ACC_COLS <= 32 ? 32 : (ACC_COLS <= 64 ? 64 : (ACC_COLS <= 128 ? 128 : (ACC_COLS <= 256 ? 256 : 512)));
    static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + INBOX_BYTES + 1024 /*alignment*/ + 1024 /*barriers*/;
};

template <int BN, bool SWIGLU>
__global__ void __launch_bounds__(THREADS)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_w2,
               const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_c,
               const GemmParams p) {
    using C = Cfg<BN, SWIGLU>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint64_t* bars = (uint64_t*)(smem + C::STAGES * C::STAGE_BYTES);
    // bars[0..S): full, bars[S..2S): empty, bars[2S]: accumulator ready
    uint32_t* tmem_slot = (uint32_t*)(bars + 2 * C::STAGES + 2);
    volatile int* give_up = (volatile int*)(tmem_slot + 1);

    pdl_launch_dependents();
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int m0 = blockIdx.x * BM, n0 = blockIdx.y * BN, split = blockIdx.z;
    const int kb0 = split * p.kb_per_split;
    const int kb1 = min(p.num_kb, kb0 + p.kb_per_split);
    const int my_kb = kb1 - kb0;
    const uint32_t full0 = smem_u32(bars), empty0 = smem_u32(bars + C::STAGES);
    const uint32_t acc_bar = smem_u32(bars + 2 * C::STAGES);
    const uint32_t inbox_bar = smem_u32(bars + 2 * C::STAGES + 1);  // counts the bytes that the cluster pushes into this CTA's inbox

    if (tid == 0) {
        for (int s = 0; s < C::STAGES; ++s) {
            mbar_init(full0 + 8 * s, 1);
            mbar_init(empty0 + 8 * s, 1);
        }
        mbar_init(acc_bar, 1);
        mbar_init(inbox_bar, 1);
        if (p.splits > 1) {
            // this CTA finishes columns [rank * per, ...) of the tile: every CTA of the cluster, itself
            // included, sends it those columns of its partial accumulator, 4 bytes per feature
            const int per0 = (BN + p.splits - 1) / p.splits;
            const int first = min(BN, (int)cluster_rank() * per0);
            const int owned = min(BN, first + per0) - first;
            mbar_expect_tx(inbox_bar, (uint32_t)(p.splits * owned * (SWIGLU ? 2 : 1) * BM * 4));
        }
        *give_up = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 2) tmem_alloc(smem_u32(tmem_slot), C::TMEM_COLS);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    // Every inbox barrier of the cluster is initialised before any CTA can push (long before: the
    // pushes come after the main loop).  This is the kernel's only cluster-wide barrier, and it falls
    // into the time before the preceding kernel has finished.
    if (p.splits > 1) cluster_sync();

    int issued = 0;
    if (warp == 0 && lane == 0) {
        // ---- TMA producer ----------------------------------------------------------------------
        // Weight tiles of the first stages go out before the wait on the preceding kernel: no
        // kernel of the step writes weights, so they stream while that kernel finishes.  The
        // activation tiles (which it may still be writing) follow after the wait.
        const int early = min(my_kb, C::STAGES);
        for (int i = 0; i < early; ++i) {
            const uint32_t a_dst = smem_u32(smem + i * C::STAGE_BYTES);
            const uint32_t bar = full0 + 8 * i;
            mbar_expect_tx(bar, C::STAGE_BYTES);
            const int kx = (kb0 + i) * BK;
            tma_load_2d(a_dst, &map_w, kx, m0, bar);
            if (SWIGLU) tma_load_2d(a_dst + C::A_BYTES, &map_w2, kx, m0, bar);
        }
        pdl_wait();
        for (int i = 0; i < early; ++i) {
            const uint32_t a_dst = smem_u32(smem + i * C::STAGE_BYTES);
            tma_load_2d(a_dst + C::A_BYTES * (SWIGLU ? 2 : 1), &map_x, (kb0 + i) * BK, n0, full0 + 8 * i);
            ++issued;
        }
        for (int i = early; i < my_kb; ++i) {
            const int s = i % C::STAGES;
            const uint32_t parity = ((i / C::STAGES) & 1) ^ 1;
            if (!mbar_wait(empty0 + 8 * s, parity, give_up)) break;
            const uint32_t a_dst = smem_u32(smem + s * C::STAGE_BYTES);
            const uint32_t bar = full0 + 8 * s;
            mbar_expect_tx(bar, C::STAGE_BYTES);
            const int kx = (kb0 + i) * BK;
            tma_load_2d(a_dst, &map_w, kx, m0, bar);
            if (SWIGLU) tma_load_2d(a_dst + C::A_BYTES, &map_w2, kx, m0, bar);
            tma_load_2d(a_dst + C::A_BYTES * (SWIGLU ? 2 : 1), &map_x, kx, n0, bar);
            ++issued;
        }
    } else if (warp == 1 && lane == 0) {
        // ---- MMA issuer ------------------------------------------------------------------------
        pdl_wait();  // blocked here a thread costs nothing; polling a barrier takes issue slots
        constexpr uint32_t idesc = instr_desc(BM, BN);
        bool ok = true;
        for (int i = 0; i < my_kb && ok; ++i) {
            const int s = i % C::STAGES;
            ok = mbar_wait(full0 + 8 * s, (i / C::STAGES) & 1, give_up);
            if (!ok) break;
            tc_fence_after();
            const uint32_t a_addr = smem_u32(smem + s * C::STAGE_BYTES);
            const uint64_t adesc = smem_desc_sw128(a_addr);
            const uint64_t a2desc = smem_desc_sw128(a_addr + C::A_BYTES);
            const uint64_t bdesc = smem_desc_sw128(a_addr + C::A_BYTES * (SWIGLU ? 2 : 1));
#pragma unroll
            for (int k = 0; k < BK / 16; ++k) {
                // 16 bf16 = 32 bytes further along K inside the swizzle atom: +2 in 16-byte units
                const uint32_t acc = (i > 0 || k > 0) ? 1u : 0u;
                umma_bf16(tmem_base, adesc + 2 * k, bdesc + 2 * k, idesc, acc);
                if (SWIGLU) umma_bf16(tmem_base + BN, a2desc + 2 * k, bdesc + 2 * k, idesc, acc);
            }
            umma_commit(empty0 + 8 * s);  // frees the stage when these MMAs have read it
        }
        if (ok) umma_commit(acc_bar);
    }
    __syncwarp();
    // ---- epilogue: every thread owns one output feature (TMEM lane) -----------------------------
    // First the wait on the preceding kernel (the epilogue reads and writes what it wrote), then every
    // load that does not depend on the accumulator: they are in flight while the main loop runs, so
    // that after the accumulator is ready nothing waits on global memory again.
    pdl_wait();
    const int row = warp * 32 + lane;  // feature within the tile
    const int f = m0 + row;
    constexpr bool NORM_OK = BN <= 128;  // the shared arrays below hold 128 tokens
    float* inv_s = (float*)((uint8_t*)bars + 256);  // [128] the tokens' 1/rms, when a norm is finished here
    float* red_s = inv_s + 128;                     // [4][16] per-warp sums of squares, when one is begun here
    const bool scaled = NORM_OK && p.scale_part != nullptr;
    const bool emit = !SWIGLU && NORM_OK && p.emit_x != nullptr && p.epilogue == 1;  // the same in the whole CTA
    const float bias = (p.bias != nullptr && f < p.N) ? p.bias[f] : 0.f;
    const float emit_gf = (emit && f < p.N) ? p.emit_g[f] : 0.f;
    // the slice of the tile's columns that this CTA finishes (all of them when the tile is not split)
    const int per = (BN + p.splits - 1) / p.splits;        // columns per owner
    const int slots = per * (SWIGLU ? 2 : 1);              // inbox column slots per sender
    const uint32_t my_rank = p.splits > 1 ? cluster_rank() : 0;
    int c_begin = p.splits > 1 ? min(BN, (int)my_rank * per) : 0;
    int c_end = p.splits > 1 ? min(BN, c_begin + per) : BN;
    // A slice of at most four columns (decode: few tokens, the inner dimension split over many CTAs)
    // is finished by a four-column form of the code below, and the residual's old values for it are
    // fetched here.  The instruction footprint matters as much as the instruction count: each CTA
    // runs its epilogue once, straight from the instruction cache's misses.
    const bool small_slice = p.splits > 1 && c_end - c_begin <= 4;
    const bool medium_slice = p.splits > 1 && c_end - c_begin <= 8;
    float old0[4] = {0.f, 0.f, 0.f, 0.f};
    if (small_slice && !SWIGLU && p.epilogue == 1 && f < p.N) {
        const float* c32 = (const float*)p.C + (size_t)(n0 + c_begin) * p.ldc + f;
#pragma unroll
        for (int j = 0; j < 4; ++j)
            if (c_begin + j < c_end && n0 + c_begin + j < p.T) old0[j] = c32[(size_t)j * p.ldc];
    }
    if (scaled && warp >= 2) {
        for (int i = tid - 64; i < BN; i += 64) {
            const int t = n0 + i;
            float ssq = 0.f;
            if (t < p.T) {
                // sixteen loads in flight at a time (a loop of one load and one add each would pay the
                // L2's latency once per term), summed in index order
                const float* part = p.scale_part + (size_t)t * p.scale_parts;
                for (int i0 = 0; i0 < p.scale_parts; i0 += 16) {
                    float v[16];
#pragma unroll
                    for (int k = 0; k < 16; ++k) v[k] = i0 + k < p.scale_parts ? part[i0 + k] : 0.f;
#pragma unroll
                    for (int k = 0; k < 16; ++k) ssq += v[k];
                }
            }
            inv_s[i] = 1.0f / sqrtf(ssq / (float)p.scale_dim + p.scale_eps);
        }
    }
    const bool acc_ready = __syncthreads_and(mbar_wait(acc_bar, 0, give_up) ? 1 : 0) != 0;  // one answer for the CTA; inv_s visible
    tc_fence_after();
    __syncwarp();
    const uint32_t taddr = tmem_base + ((uint32_t)(warp * 32) << 16);
    // With the inner dimension split, the CTAs of one tile form a cluster and each finishes a slice of
    // the tile's columns.  A CTA pushes every column of its partial accumulator into the inbox of the
    // column's owner (st.async into distributed shared memory, slot = sender's rank; each store adds
    // its 4 bytes to the owner's inbox barrier), and each owner waits for its own inbox only, then adds
    // the partials it received in rank order.  Nobody waits for the whole cluster, and a CTA whose
    // inbox is complete touches nobody else's memory again, so CTAs leave independently.
    float* stage = (float*)smem;  // unsplit tiles: [token][feature] staging for the TMA store
    const uint32_t stage_addr = smem_u32(stage);
    float* inbox = (float*)(smem + C::STAGES * C::STAGE_BYTES + 1024);  // [rank][column slot][BM]
    if (p.splits > 1) {
        const uint32_t inbox_addr = smem_u32(inbox);
        int owner = 0, local = 0;
        for (int c = 0; c < BN; c += 16) {
            float v[16], v2[16];
            if (acc_ready) {
                tmem_ld16(taddr + c, v);
                if (SWIGLU) tmem_ld16(taddr + BN + c, v2);
            } else {
#pragma unroll
                for (int j = 0; j < 16; ++j) v[j] = v2[j] = 0.f;
            }
#pragma unroll
            for (int j = 0; j < 16; ++j) {
                // column c + j belongs to `owner`, as its column `local` (counted up: no division here)
                const uint32_t a = dsmem_addr(inbox_addr + (uint32_t)(((my_rank * slots + local) * BM + row) * 4), owner);
                const uint32_t b = dsmem_addr(inbox_bar, owner);
                st_async_dsmem(a, v[j], b);
                if (SWIGLU) st_async_dsmem(a + (uint32_t)(per * BM * 4), v2[j], b);
                if (++local == per) {
                    local = 0;
                    ++owner;
                }
            }
        }
        if (c_end > c_begin) mbar_wait(inbox_bar, 0, give_up);  // (a timeout is reported at teardown)
    }
    if (p.splits == 1 && p.tma_store && acc_ready) {
        // The whole tile goes to shared memory as [token][feature] in C's type, then leaves in one
        // TMA store (or float32 reduce-add into the residual): full-line writes, no read-modify-write
        // round trips from the SM, and no per-element address arithmetic.
        const bool wide = !SWIGLU && p.epilogue != 0;  // float32 C
        for (int c = 0; c < BN; c += 16) {
            float g[16], u[16];
            tmem_ld16(taddr + c, g);
            if (SWIGLU) tmem_ld16(taddr + BN + c, u);
#pragma unroll
            for (int j = 0; j < 16; ++j) {
                const float sc = scaled ? inv_s[c + j] : 1.0f;
                float v = g[j] * sc + bias;
                if (SWIGLU) v = __fdividef(v, 1.0f + __expf(-v)) * (u[j] * sc);
                if (wide)
                    stage[(c + j) * BM + row] = v;
                else
                    ((bf16*)stage)[(c + j) * BM + row] = __float2bfloat16_rn(v);
            }
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // generic-proxy writes -> TMA
        __syncthreads();
        if (tid == 0) tma_store_2d(&map_c, stage_addr, m0, n0, !SWIGLU && p.epilogue == 1);
        c_begin = c_end = 0;  // nothing left for the direct path
    }
    auto finish = [&](auto width) {
        constexpr int NC = decltype(width)::value;  // columns per pass: 4 (small slices) or 16
        for (int c = c_begin; c < c_end && (acc_ready || p.splits > 1); c += NC) {
            const int ncols = min(NC, c_end - c);
            float g[NC], u[NC];
            if (NC == 16 && p.splits == 1) {
                float g16[16], u16[16];
                tmem_ld16(taddr + c, g16);
                if (SWIGLU) tmem_ld16(taddr + BN + c, u16);
#pragma unroll
                for (int j = 0; j < NC; ++j) {
                    g[j] = g16[j & 15];
                    u[j] = SWIGLU ? u16[j & 15] : 0.f;
                }
            } else {
#pragma unroll
                for (int j = 0; j < NC; ++j) g[j] = u[j] = 0.f;
                for (int s = 0; s < p.splits; ++s) {  // rank order; all reads are of this CTA's own inbox
                    const float* part = inbox + ((size_t)s * slots + (c - c_begin)) * BM + row;
#pragma unroll
                    for (int j = 0; j < NC; ++j) {
                        if (j < ncols) {
                            g[j] += part[j * BM];
                            if (SWIGLU) u[j] += part[(per + j) * BM];
                        }
                    }
                }
            }
            const int t_base = n0 + c;
            float sq[NC];
#pragma unroll
            for (int j = 0; j < NC; ++j) {
                sq[j] = 0.f;
                const float sc = scaled ? inv_s[(c + j) & (BN - 1)] : 1.0f;
                g[j] = g[j] * sc + bias;
                if (SWIGLU) u[j] *= sc;
            }
            // one loop per kind of epilogue (not one loop with the kinds inside): only the one that runs
            // is fetched.  The columns are independent and the loops straight-line, so that the
            // compiler interleaves their arithmetic.
            if (f < p.N) {
                float* c32 = (float*)p.C + (size_t)t_base * p.ldc + f;
                bf16* c16 = (bf16*)p.C + (size_t)t_base * p.ldc + f;
                if (SWIGLU) {
                    // silu(v) * u with the fast exponential and division: the result is rounded to
                    // bfloat16 (8 bits) right after, their 2^-21 relative error does not show
#pragma unroll
                    for (int j = 0; j < NC; ++j)
                        if (j < ncols && t_base + j < p.T)
                            c16[(size_t)j * p.ldc] = __float2bfloat16_rn(__fdividef(g[j], 1.0f + __expf(-g[j])) * u[j]);
                } else if (p.epilogue == 0) {
#pragma unroll
                    for (int j = 0; j < NC; ++j)
                        if (j < ncols && t_base + j < p.T) c16[(size_t)j * p.ldc] = __float2bfloat16_rn(g[j]);
                } else if (p.epilogue == 1) {
                    float old[NC];
                    // all loads first: issued back to back instead of one load-add-store chain each
#pragma unroll
                    for (int j = 0; j < NC; ++j) {
                        if (NC == 4)
                            old[j] = old0[j & 3];  // fetched before the accumulator was ready
                        else
                            old[j] = (j < ncols && t_base + j < p.T) ? c32[(size_t)j * p.ldc] : 0.f;
                    }
#pragma unroll
                    for (int j = 0; j < NC; ++j) {
                        const float nv = old[j] + g[j];
                        if (j < ncols && t_base + j < p.T) {
                            c32[(size_t)j * p.ldc] = nv;
                            if (emit) {
                                p.emit_x[(size_t)(t_base + j) * p.N + f] = __float2bfloat16_rn(nv * emit_gf);
                                sq[j] = nv * nv;
                            }
                        }
                    }
                } else {
#pragma unroll
                    for (int j = 0; j < NC; ++j)
                        if (j < ncols && t_base + j < p.T) c32[(size_t)j * p.ldc] = g[j];
                }
            }
            if (emit) {
                // the tile's share of each token's sum of squares: over the warp, then over the four warps
#pragma unroll
                for (int j = 0; j < NC; ++j) {
                    const float w = warp_sum(sq[j]);
                    if (lane == 0) red_s[warp * 16 + j] = w;
                }
                __syncthreads();
                if (tid < ncols && t_base + tid < p.T)
                    p.emit_part[(size_t)(t_base + tid) * gridDim.x + blockIdx.x] =
                        (red_s[tid] + red_s[16 + tid]) + (red_s[32 + tid] + red_s[48 + tid]);
                __syncthreads();
            }
        }
    };
    if (small_slice)
        finish(std::integral_constant<int, 4>{});
    else if (medium_slice)
        finish(std::integral_constant<int, 8>{});
    else
        finish(std::integral_constant<int, 16>{});
    // ---- teardown ---------------------------------------------------------------------------------
    if (*give_up) {
        if (tid == 0) cw_report(p.status, CW_ST_WAIT_TIMEOUT, blockIdx.x, blockIdx.z);
        if (warp == 0 && lane == 0) {
            // wait, bounded, for the copies still in flight before the CTA's shared memory goes away
            for (int i = max(0, issued - C::STAGES); i < issued; ++i) {
                const uint32_t bar = full0 + 8 * (i % C::STAGES);
                const long long t0 = clock64();
                while (!mbar_try_wait(bar, (i / C::STAGES) & 1) && clock64() - t0 < WAIT_CYCLES) {
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 2) tmem_dealloc(tmem_base, C::TMEM_COLS);
    cw_trace_end();
}

// ---------------------------------------------------------------------------------------------
// Persistent form for large problems (more output tiles than SMs, no split): one CTA per SM walks
// tiles; the accumulator is double-buffered in TMEM so that the epilogue of one tile (TMEM ->
// registers -> shared memory -> TMA store / reduce-add, 16 tokens at a time) runs while the MMAs of
// the next tile proceed.  Warps: 0 TMA producer, 1 MMA issuer and TMEM owner, 2..5 epilogue.
// ---------------------------------------------------------------------------------------------
#define P_THREADS 192
#define P_CHUNK 16  // tokens per epilogue store
#define MAX_SMEM_BYTES (227 * 1024)

template <int BN, bool SWIGLU>
struct PCfg {
    static constexpr int A_BYTES = BM * BK * 2;
    static constexpr int B_BYTES = BN * BK * 2;
    static constexpr int STAGE_BYTES = A_BYTES * (SWIGLU ? 2 : 1) + B_BYTES;
    static constexpr int ACC_COLS = BN * (SWIGLU ? 2 : 1);
    static constexpr int TMEM_COLS = 2 * ACC_COLS <= 256 ? 256 : 512;
    static constexpr int OUT_BYTES = 2 * P_CHUNK * BM * 4;  // two staging buffers of [16 tokens][128 features]
    static constexpr int STAGES = (MAX_SMEM_BYTES - 2048 - OUT_BYTES) / STAGE_BYTES;
    static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + OUT_BYTES + 1024 + 1024;
    static_assert(2 * ACC_COLS <= 512, "two accumulators must fit in tensor memory");
    static_assert(STAGES >= 3, "too few operand stages");
};

template <int BN, bool SWIGLU>
__global__ void __launch_bounds__(P_THREADS, 1)
gemm_tc_persistent_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_w2,
                          const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_c,
                          const GemmParams p) {
    using C = PCfg<BN, SWIGLU>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t* out_s = smem + C::STAGES * C::STAGE_BYTES;
    uint64_t* bars = (uint64_t*)(out_s + C::OUT_BYTES);
    // bars: full[S], empty[S], acc_full[2], acc_empty[2]
    uint32_t* tmem_slot = (uint32_t*)(bars + 2 * C::STAGES + 4);
    volatile int* give_up = (volatile int*)(tmem_slot + 1);

    // Only the activations come from the preceding kernel, and only the producer thread reads them
    // (everything else follows from its copies): it alone waits for that kernel, after the set-up and
    // after the weight tiles of the first stages have gone out.
    pdl_launch_dependents();
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t full0 = smem_u32(bars), empty0 = smem_u32(bars + C::STAGES);
    const uint32_t accf0 = smem_u32(bars + 2 * C::STAGES), acce0 = smem_u32(bars + 2 * C::STAGES + 2);
    const int bn = p.bn;  // <= BN; the accumulators keep their places for the widest tile
    const int m_tiles = (p.N + BM - 1) / BM, n_tiles = (p.T + bn - 1) / bn;
    const uint32_t stage_tx = C::A_BYTES * (SWIGLU ? 2 : 1) + bn * BK * 2;
    const int tiles = m_tiles * n_tiles;

    if (tid == 0) {
        for (int s = 0; s < C::STAGES; ++s) {
            mbar_init(full0 + 8 * s, 1);
            mbar_init(empty0 + 8 * s, 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(accf0 + 8 * b, 1);
            mbar_init(acce0 + 8 * b, 1);
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

    if (warp == 0 && lane == 0) {
        // ---- TMA producer: runs ahead over tiles, bounded by the ring only ----------------------------
        const int my_tiles = (int)blockIdx.x < tiles ? (tiles - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x : 0;
        const int total = my_tiles * p.num_kb;  // k-blocks of all this CTA's tiles, in order
        const int early = min(total, C::STAGES);
        int i = 0;
        bool ok = true;
        // the first stages: weight tiles before the wait, their activation tiles after it
        for (int phase = 0; phase < 2; ++phase) {
            if (phase == 1) pdl_wait();
            for (i = 0; i < early; ++i) {
                const int ts = i / p.num_kb, kb = i - ts * p.num_kb, tile = blockIdx.x + ts * gridDim.x;
                const int m0 = (tile % m_tiles) * BM, n0 = (tile / m_tiles) * bn;
                const uint32_t a_dst = smem_u32(smem + i * C::STAGE_BYTES);
                const uint32_t bar = full0 + 8 * i;
                if (phase == 0) {
                    mbar_expect_tx(bar, stage_tx);
                    tma_load_2d(a_dst, &map_w, kb * BK, m0, bar);
                    if (SWIGLU) tma_load_2d(a_dst + C::A_BYTES, &map_w2, kb * BK, m0, bar);
                } else {
                    tma_load_2d(a_dst + C::A_BYTES * (SWIGLU ? 2 : 1), &map_x, kb * BK, n0, bar);
                }
            }
        }
        // the rest runs ahead over tiles, bounded by the ring only
        int kb = early % p.num_kb;
        for (int tile = blockIdx.x + (early / p.num_kb) * gridDim.x; tile < tiles && ok; tile += gridDim.x, kb = 0) {
            const int m0 = (tile % m_tiles) * BM, n0 = (tile / m_tiles) * bn;
            for (; kb < p.num_kb; ++kb, ++i) {
                const int s = i % C::STAGES;
                ok = mbar_wait(empty0 + 8 * s, ((i / C::STAGES) & 1) ^ 1, give_up);
                if (!ok) break;
                const uint32_t a_dst = smem_u32(smem + s * C::STAGE_BYTES);
                const uint32_t bar = full0 + 8 * s;
                mbar_expect_tx(bar, stage_tx);
                tma_load_2d(a_dst, &map_w, kb * BK, m0, bar);
                if (SWIGLU) tma_load_2d(a_dst + C::A_BYTES, &map_w2, kb * BK, m0, bar);
                tma_load_2d(a_dst + C::A_BYTES * (SWIGLU ? 2 : 1), &map_x, kb * BK, n0, bar);
            }
        }
        if (*give_up) {
            // wait, bounded, for the copies still in flight before the CTA's shared memory goes away
            for (int k = max(0, i - C::STAGES); k < i; ++k) {
                const uint32_t bar = full0 + 8 * (k % C::STAGES);
                const long long t0 = clock64();
                while (!mbar_try_wait(bar, (k / C::STAGES) & 1) && clock64() - t0 < WAIT_CYCLES) {
                }
            }
        }
    } else if (warp == 1 && lane == 0) {
        // ---- MMA issuer: tile `it` accumulates into TMEM buffer it & 1 -------------------------------
        pdl_wait();  // (nothing to do before the producer's activations arrive; parked here a thread polls no barrier)
        const uint32_t idesc = instr_desc(BM, bn);
        int i = 0, it = 0;
        bool ok = true;
        for (int tile = blockIdx.x; tile < tiles && ok; tile += gridDim.x, ++it) {
            const int buf = it & 1;
            ok = mbar_wait(acce0 + 8 * buf, ((it >> 1) & 1) ^ 1, give_up);  // the epilogue has drained it
            if (!ok) break;
            tc_fence_after();
            const uint32_t acc = tmem_base + buf * C::ACC_COLS;
            for (int kb = 0; kb < p.num_kb; ++kb, ++i) {
                const int s = i % C::STAGES;
                ok = mbar_wait(full0 + 8 * s, (i / C::STAGES) & 1, give_up);
                if (!ok) break;
                tc_fence_after();
                const uint32_t a_addr = smem_u32(smem + s * C::STAGE_BYTES);
                const uint64_t adesc = smem_desc_sw128(a_addr);
                const uint64_t a2desc = smem_desc_sw128(a_addr + C::A_BYTES);
                const uint64_t bdesc = smem_desc_sw128(a_addr + C::A_BYTES * (SWIGLU ? 2 : 1));
#pragma unroll
                for (int k = 0; k < BK / 16; ++k) {
                    const uint32_t accumulate = (kb > 0 || k > 0) ? 1u : 0u;
                    umma_bf16(acc, adesc + 2 * k, bdesc + 2 * k, idesc, accumulate);
                    if (SWIGLU) umma_bf16(acc + BN, a2desc + 2 * k, bdesc + 2 * k, idesc, accumulate);
                }
                umma_commit(empty0 + 8 * s);
            }
            if (ok) umma_commit(accf0 + 8 * buf);
        }
    } else if (warp >= 2) {
        // ---- epilogue warps: warp w reads TMEM lanes 32 (w % 4) .. +31 -------------------------------
        pdl_wait();
        const int quarter = warp & 3;
        const int row = quarter * 32 + lane;
        const int etid = tid - 64;  // 0..127 among the epilogue threads
        const bool wide = !SWIGLU && p.epilogue != 0;
        int it = 0, chunk_no = 0;
        bool ok = true;
        for (int tile = blockIdx.x; tile < tiles && ok; tile += gridDim.x, ++it) {
            const int buf = it & 1;
            const int m0 = (tile % m_tiles) * BM, n0 = (tile / m_tiles) * bn;
            const int f = m0 + row;
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
            const uint32_t taddr = tmem_base + buf * C::ACC_COLS + ((uint32_t)(quarter * 32) << 16);
            const float bias = (p.bias != nullptr && f < p.N) ? p.bias[f] : 0.f;
            // Only chunks that hold tokens are read out and stored.  Every chunk that runs issues exactly one
            // store and one bulk group, so that `wait_group.read 1` below means what it says: the store that
            // read this staging buffer two chunks ago is done with it.  (A chunk that skipped its store but
            // still filled the buffer would overwrite what the store of two chunks ago may still be reading.)
            const int c_end = min(bn, p.T - n0);
            for (int c = 0; c < c_end; c += P_CHUNK, ++chunk_no) {
                float g[16], u[16];
                tmem_ld16(taddr + c, g);
                if (SWIGLU) tmem_ld16(taddr + BN + c, u);
                if (c + P_CHUNK >= c_end) {
                    // the accumulator has been read out: hand the buffer back to the MMA warp
                    tc_fence_before();
                    asm volatile("bar.sync 1, 128;" ::: "memory");
                    if (etid == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(acce0 + 8 * buf) : "memory");
                }
                float* st32 = (float*)(out_s + (chunk_no & 1) * (C::OUT_BYTES / 2));
                // the store that used this staging buffer two chunks ago must have read it
                if (etid == 0) asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
                asm volatile("bar.sync 2, 128;" ::: "memory");
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                    float v = g[j] + bias;
                    if (SWIGLU) v = __fdividef(v, 1.0f + __expf(-v)) * u[j];
                    if (wide)
                        st32[j * BM + row] = v;
                    else
                        ((bf16*)st32)[j * BM + row] = __float2bfloat16_rn(v);
                }
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                asm volatile("bar.sync 1, 128;" ::: "memory");
                if (etid == 0) {
                    const bool add = !SWIGLU && p.epilogue == 1;
                    if (add)
                        asm volatile("cp.reduce.async.bulk.tensor.2d.global.shared::cta.add.bulk_group [%0, {%2, %3}], [%1];"
                                     ::"l"(&map_c), "r"(smem_u32(st32)), "r"(m0), "r"(n0 + c) : "memory");
                    else
                        asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
                                     ::"l"(&map_c), "r"(smem_u32(st32)), "r"(m0), "r"(n0 + c) : "memory");
                    asm volatile("cp.async.bulk.commit_group;" ::: "memory");
                }
            }
        }
        if (etid == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");  // all stores done before exit
    }
    __syncwarp();
    if (*give_up && tid == 0) cw_report(p.status, CW_ST_WAIT_TIMEOUT, blockIdx.x, -1);
    tc_fence_before();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem_base, C::TMEM_COLS);
}

// ---------------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------------
// A [rows, K] bf16 matrix with row stride `ld` elements, read in boxes of `box_rows` x 64.
static int make_map(CUtensorMap* map, const void* ptr, int rows, int K, long long ld, int box_rows) {
    const cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
    const cuuint32_t box[2] = {BK, (cuuint32_t)box_rows};
    const cuuint32_t elem[2] = {1, 1};
    const CUresult r = g_encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides,
                                box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : -1;
}

// C [T, N] (row stride ldc elements) written in boxes of `box_rows` tokens x 128 features, no swizzle.
static int make_map_c(CUtensorMap* map, const void* ptr, int T, int N, long long ldc, int box_rows, bool f32) {
    const cuuint64_t dims[2] = {(cuuint64_t)N, (cuuint64_t)T};
    const cuuint64_t strides[1] = {(cuuint64_t)ldc * (f32 ? 4 : 2)};
    const cuuint32_t box[2] = {BM, (cuuint32_t)box_rows};
    const cuuint32_t elem[2] = {1, 1};
    const CUresult r = g_encode(map, f32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2,
                                const_cast<void*>(ptr), dims, strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE,
                                CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_NONE,
                                CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : -1;
}

struct Plan {
    int bn, splits, kb_per_split, tiles;
    bool persistent;  // bn is then any multiple of 16 and the persistent kernel runs
    bool pair;        // ... on CTA pairs: tiles of 256 features
    bool stream;      // few tokens, many rounds of weight tiles (a vocabulary): the persistent kernel with narrow tiles
};

// Token-tile width for CTA pairs: per k-block a pair-tile costs about max(2 bn, 256 + bn) cycles (MMA
// time, shared-memory traffic) and the pairs run ceil(tiles / pairs) rounds.
static int balanced_bn_pair(int T, int N, int sm_count, bool swiglu = false) {
    const int m_tiles = (N + 2 * BM - 1) / (2 * BM), pairs = sm_count / 2;
    long long best_cost = -1;
    const int cap = swiglu ? 128 : 256;  // (SwiGLU: two accumulators per tile, two weight tiles per k-block)
    int best = cap;
    for (int bn = cap; bn >= 64; bn -= 16) {
        const long long tiles = (long long)m_tiles * ((T + bn - 1) / bn);
        const long long rounds = (tiles + pairs - 1) / pairs;
        const long long cost = swiglu ? rounds * (4 * bn > 512 + bn ? 4 * bn : 512 + bn)
                                      : rounds * (2 * bn > 256 + bn ? 2 * bn : 256 + bn);
        if (best_cost < 0 || cost < best_cost) {
            best_cost = cost;
            best = bn;
        }
    }
    return best;
}

// Token-tile width for the persistent kernel.  A k-block costs a tile about 256 + 2 bn cycles of
// shared-memory traffic (the weight tile is loaded whatever bn is, SwiGLU loads two) and the CTAs
// run ceil(tiles / SMs) rounds; the width with the least rounds x cost wins, the wider on a tie.
static int balanced_bn(int T, int N, bool swiglu, int sm_count) {
    const int cap = swiglu ? 128 : 256;
    const int m_tiles = (N + BM - 1) / BM;
    long long best_cost = -1;
    int best = cap;
    for (int bn = cap; bn >= 64; bn -= 16) {
        const long long tiles = (long long)m_tiles * ((T + bn - 1) / bn);
        const long long rounds = (tiles + sm_count - 1) / sm_count;
        const long long cost = rounds * ((swiglu ? 512 : 256) + 2 * bn);
        if (best_cost < 0 || cost < best_cost) {
            best_cost = cost;
            best = bn;
        }
    }
    return best;
}

static int g_pair_enabled = 1;
static int g_pair_swiglu = 0;
// Whether the SwiGLU product of prompt portions runs on CTA pairs too.  Off: measured equal to the
// single-CTA persistent kernel within 2 % from 256 to 4,096 tokens (under the power cap the product's
// rate is a matter of energy per FLOP, not of shared-memory traffic per tile).
extern "C" int cw_gemm_tc_set_pair_swiglu(int on) { g_pair_swiglu = on ? 1 : 0; return CW_OK; }
static int g_forced_bn = 0;
static int* g_split_flags = nullptr;  // device words for the CTA-pair kernel's split products (zero between launches)
static int g_split_flags_n = 0;
// Gives the CTA-pair kernel the device memory through which the splits of a tile take turns (n int32
// words, zeroed by the caller once; the kernel leaves them zero).  Without it no product is split.
extern "C" int cw_gemm_tc_set_split_flags(int* words, int n) {
    g_split_flags = words;
    g_split_flags_n = words != nullptr ? n : 0;
    return CW_OK;
}

// How many ways the inner dimension of a CTA-pair product that adds into its output is split: as many
// as leave no pair idle, dividing the k-blocks evenly, at least 16 k-blocks each, at most 8.
static int pair_splits(int tiles, int num_kb, int sm_count) {
    const int pairs = sm_count / 2;
    if (g_split_flags == nullptr || 2 * tiles > g_split_flags_n || tiles * 2 > pairs) return 1;
    int best = 1;
    for (int d = 2; d <= 8 && d * tiles <= pairs; ++d)
        if (num_kb % d == 0 && num_kb / d >= 16) best = d;
    return best;
}

// Token-tile width for a CTA-pair product that may be split over K.  Measured: a pair's k-block costs
// about 330 + 0.2 bn nanoseconds whatever the tile's width (the stages in flight bound it), and the
// splits of a tile store one after the other, each taking about 1000 + 25 bn nanoseconds (a turn of
// the flag, bn / 16 chunks of stores).
static int balanced_bn_pair_split(int T, int N, int num_kb, int sm_count) {
    const int m_tiles = (N + 2 * BM - 1) / (2 * BM), pairs = sm_count / 2;
    long long best_cost = -1;
    int best = 256;
    for (int bn = 256; bn >= 64; bn -= 16) {
        const int tiles = m_tiles * ((T + bn - 1) / bn);
        const int splits = pair_splits(tiles, num_kb, sm_count);
        const long long rounds = ((long long)tiles * splits + pairs - 1) / pairs;
        const long long cost = rounds * (num_kb / splits) * (330 + bn / 5) + splits * (1000LL + 25 * bn);
        if (best_cost < 0 || cost < best_cost) {
            best_cost = cost;
            best = bn;
        }
    }
    return best;
}
// A product whose splits over K are kept apart (epilogue 3): every split stores its partial tile in a
// slab of its own and whoever reads the result next adds the slabs, in split order (the RMSNorm that
// follows a product into the residual reads the residual anyway).  Nothing takes turns, so splits may
// outnumber the pairs and run in rounds.  Cost as measured for the CTA-pair kernel: a k-block about
// 330 + 0.2 bn ns, a tile's store 1000 + 25 bn ns once, and each further slab costs its reader about
// T N / 500 ns (its bytes, written and read again).
// Measured in the step (Qwen2.5-1.5B sizes, K = 8,960): 15 % of a 256-token prompt's time, 10 % at 512, 4 % at
// 1,024; from 1,056 tokens on the slabs cost what the splits save (a mixed step of 1,056 tokens 5 % slower),
// so longer products add into their output with splits that take turns, as before.
#define PARTS_MAX_TOKENS 1024
static void parts_plan(int T, int N, int K, int sm_count, int* splits_out, int* bn_out) {
    const int m_tiles = (N + 2 * BM - 1) / (2 * BM), pairs = sm_count / 2, num_kb = (K + BK - 1) / BK;
    long long best_cost = -1;
    int best_d = 1, best_bn = 256;
    for (int bn = 256; bn >= 64; bn -= 16) {
        const int tiles = m_tiles * ((T + bn - 1) / bn);
        for (int d = 1; d <= 8; ++d) {
            if (num_kb % d != 0 || (d > 1 && num_kb / d < 8)) continue;
            const long long rounds = ((long long)tiles * d + pairs - 1) / pairs;
            const long long cost = rounds * (num_kb / d) * (330 + bn / 5) + 1000 + 25 * bn + (long long)(d - 1) * T * N / 500;
            if (best_cost < 0 || cost < best_cost) {
                best_cost = cost;
                best_d = d;
                best_bn = bn;
            }
        }
    }
    *splits_out = best_d;
    *bn_out = best_bn;
}

// Forces the token-tile width of the prompt-portion kernels (0: chosen automatically); for measurements.
extern "C" int cw_gemm_tc_set_tile(int bn) {
    if (bn != 0 && (bn < 64 || bn > 256 || bn % 16 != 0)) return CW_ERR_BAD_SIZE;
    g_forced_bn = bn;
    return CW_OK;
}
// Switches the CTA-pair kernel off or on (measurements, tests of the single-CTA persistent kernel).
extern "C" int cw_gemm_tc_set_pair(int on) { g_pair_enabled = on ? 1 : 0; return CW_OK; }
static int g_stream_enabled = 1;
// Switches the persistent form of few-token products over very many weight tiles off or on (measurements).
extern "C" int cw_gemm_tc_set_stream(int on) { g_stream_enabled = on ? 1 : 0; return CW_OK; }

static int g_persistent_from = 129;
// From how many tokens on the persistent kernels run (measurements; the default is the measured crossover).
extern "C" int cw_gemm_tc_set_persistent_from(int tokens) {
    if (tokens < 129) return CW_ERR_BAD_SIZE;
    g_persistent_from = tokens;
    return CW_OK;
}

static Plan make_plan(int T, int N, int K, bool swiglu, int sm_count, bool c_by_tma = true, bool adds = false) {
    Plan pl;
    pl.persistent = T >= g_persistent_from && sm_count > 0 && c_by_tma;  // its epilogue has no other way out than TMA
    // (token tiles of the one-tile-per-CTA kernel are at most 128 wide: wider ones cannot be split over K,
    // and a product of a few hundred tokens has too few tiles to do without)
    pl.bn = T <= 16 ? 16 : (T <= 32 ? 32 : (T <= 64 ? 64 : 128));
    pl.pair = pl.persistent && (!swiglu || g_pair_swiglu) && sm_count >= 2 && g_pair_enabled;
    // Few tokens against so many weight tiles that one CTA per tile would run in three rounds or more
    // (the logits product): one CTA per SM walks the tiles instead, its loads running on into the
    // next tile while the epilogue of the last one drains, and no round is left part-filled.
    pl.stream = !pl.persistent && !swiglu && T <= 64 && sm_count > 0 && c_by_tma &&
                (long long)((N + BM - 1) / BM) >= 3LL * sm_count && g_stream_enabled;
    if (pl.stream) pl.persistent = true;
    if (pl.persistent && !pl.stream) pl.bn = pl.pair ? balanced_bn_pair(T, N, sm_count, swiglu) : balanced_bn(T, N, swiglu, sm_count);
    if (pl.persistent && !pl.stream && g_forced_bn != 0 && (!swiglu || g_forced_bn <= 128)) pl.bn = g_forced_bn;
    pl.tiles = pl.pair ? ((N + 2 * BM - 1) / (2 * BM)) * ((T + pl.bn - 1) / pl.bn) : ((N + BM - 1) / BM) * ((T + pl.bn - 1) / pl.bn);
    const int num_kb = (K + BK - 1) / BK;
    int splits = 1;
    const bool can_split = pl.bn <= 64 || (pl.bn == 128 && !swiglu);  // Cfg::CAN_SPLIT
    if (!pl.persistent && can_split && pl.tiles * 2 <= sm_count) {
        // One wave: as many CTAs as SMs at most, each with as much of K as possible.  A CTA costs a
        // few microseconds of set-up and epilogue whatever it streams, so fewer, longer CTAs win
        // as long as every SM has one.
        splits = sm_count / pl.tiles;
        const int max_by_k = num_kb / 4 > 0 ? num_kb / 4 : 1;
        if (splits > max_by_k) splits = max_by_k;
        if (splits > MAX_SPLITS) splits = MAX_SPLITS;
        if (splits < 1) splits = 1;
    }
    pl.kb_per_split = (num_kb + splits - 1) / splits;
    pl.splits = (num_kb + pl.kb_per_split - 1) / pl.kb_per_split;  // no empty split
    if (pl.pair && adds && g_forced_bn == 0) {
        // products that add into their output may be split over K when the tiles leave pairs idle
        pl.bn = balanced_bn_pair_split(T, N, num_kb, sm_count);
        pl.tiles = ((N + 2 * BM - 1) / (2 * BM)) * ((T + pl.bn - 1) / pl.bn);
    }
    if (pl.pair && adds) {
        pl.splits = pair_splits(pl.tiles, num_kb, sm_count);
        pl.kb_per_split = num_kb / pl.splits;
    }
    return pl;
}

template <int BN, bool SWIGLU>
static int launch(const CUtensorMap& mw, const CUtensorMap& mw2, const CUtensorMap& mx, const CUtensorMap& mc,
                  const GemmParams& p, dim3 grid, cudaStream_t stream) {
    using C = Cfg<BN, SWIGLU>;
    static_assert(C::ACC_COLS * BM * 4 <= C::STAGES * C::STAGE_BYTES, "a staged tile must fit in the operand stages");
    static_assert(C::STAGES >= 2, "too few operand stages");
    if (grid.z > 1 && !C::CAN_SPLIT) return CW_ERR_UNSUPPORTED;
    static bool configured = false;
    if (!configured) {
        if (cudaFuncSetAttribute(gemm_tc_kernel<BN, SWIGLU>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 C::SMEM_BYTES) != cudaSuccess)
            return (int)cudaGetLastError();
        configured = true;
    }
    return cw_launch(gemm_tc_kernel<BN, SWIGLU>, grid, dim3(THREADS), C::SMEM_BYTES, stream, grid.z, mw, mw2, mx, mc, p);
}

template <bool SWIGLU>
static int launch_pair(const CUtensorMap& mw, const CUtensorMap& mw2, const CUtensorMap& mx, const CUtensorMap& mc,
                       const GemmParams& p, int pairs, cudaStream_t stream) {
    using C = PairCfgT<SWIGLU>;
    static bool configured = false;
    if (!configured) {
        if (cudaFuncSetAttribute(gemm_tc_pair_kernel<SWIGLU>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES) != cudaSuccess)
            return (int)cudaGetLastError();
        configured = true;
    }
    return cw_launch(gemm_tc_pair_kernel<SWIGLU>, dim3(2 * pairs), dim3(PAIR_THREADS), C::SMEM_BYTES, stream, 1, mw, mw2, mx, mc, p);
}

template <int BN, bool SWIGLU>
static int launch_persistent(const CUtensorMap& mw, const CUtensorMap& mw2, const CUtensorMap& mx,
                             const CUtensorMap& mc, const GemmParams& p, int ctas, cudaStream_t stream) {
    using C = PCfg<BN, SWIGLU>;
    static bool configured = false;
    if (!configured) {
        if (cudaFuncSetAttribute(gemm_tc_persistent_kernel<BN, SWIGLU>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 C::SMEM_BYTES) != cudaSuccess)
            return (int)cudaGetLastError();
        configured = true;
    }
    return cw_launch(gemm_tc_persistent_kernel<BN, SWIGLU>, dim3(ctas), dim3(P_THREADS), C::SMEM_BYTES, stream, 1, mw, mw2,
                     mx, mc, p);
}

// How a call would be tiled: token tile, splits of the inner dimension (= cluster size), CTAs.
extern "C" int cw_gemm_tc_plan(int T, int N, int K, int swiglu, int sm_count, int* bn, int* splits, int* ctas) {
    const Plan pl = make_plan(T, N, K, swiglu != 0, sm_count);
    *bn = pl.bn;
    *splits = pl.splits;
    *ctas = pl.pair ? 2 * pl.tiles * pl.splits : pl.tiles * pl.splits;
    return CW_OK;
}

// X [T, K] (row stride ldx), W [N, K] (and W2 for SwiGLU), C [T, ldc].  K must be a multiple of 8
// and all bases 16-byte aligned (TMA); returns CW_ERR_UNSUPPORTED otherwise so the caller can
// use the plain kernel.
//
// The `_norm` form splits an RMSNorm over two products (see GemmParams): with `scale_part` this
// product finishes a norm whose un-normalised, weight-multiplied rows it got as X; with `emit_x`
// (epilogue 1 only) it begins the norm that follows it.  Both need at most 128 tokens
// (CW_ERR_UNSUPPORTED otherwise).
extern "C" int cw_gemm_tc_norm(const void* X, const void* W, const void* W2, const float* bias, void* C, int T,
                               int N, int K, int ldx, int ldc, int epilogue, int sm_count,
                               const float* scale_part, int scale_parts, float scale_eps, int scale_dim,
                               const float* emit_g, void* emit_x, float* emit_part, int* status,
                               cudaStream_t stream);

extern "C" int cw_gemm_tc(const void* X, const void* W, const void* W2, const float* bias, void* C, int T,
                          int N, int K, int ldx, int ldc, int epilogue, int sm_count, int* status,
                          cudaStream_t stream) {
    return cw_gemm_tc_norm(X, W, W2, bias, C, T, N, K, ldx, ldc, epilogue, sm_count, nullptr, 0, 0.f, 1, nullptr,
                           nullptr, nullptr, status, stream);
}

extern "C" int cw_gemm_tc_norm(const void* X, const void* W, const void* W2, const float* bias, void* C, int T,
                               int N, int K, int ldx, int ldc, int epilogue, int sm_count,
                               const float* scale_part, int scale_parts, float scale_eps, int scale_dim,
                               const float* emit_g, void* emit_x, float* emit_part, int* status,
                               cudaStream_t stream) {
    if (T == 0 || N == 0) return CW_OK;
    if (T < 0 || N < 0 || K <= 0 || ldx < K || ldc < N) return CW_ERR_BAD_SIZE;
    if (epilogue < 0 || epilogue > 2) return CW_ERR_UNSUPPORTED;
    if (K % 8 != 0 || ldx % 8 != 0 || ((uintptr_t)X & 15) || ((uintptr_t)W & 15) || ((uintptr_t)W2 & 15))
        return CW_ERR_UNSUPPORTED;
    if (load_encode() != 0) return CW_ERR_UNSUPPORTED;
    const bool swiglu = W2 != nullptr;
    // C leaves through TMA when its rows are 16-byte multiples at a 16-byte base and the tile is not split
    const bool c_f32 = !swiglu && epilogue != 0;
    const long long c_row_bytes = (long long)ldc * (c_f32 ? 4 : 2);
    const bool c_by_tma = c_row_bytes % 16 == 0 && ((uintptr_t)C & 15) == 0;
    const bool emits = emit_x != nullptr;
    // (a product that finishes or begins a norm has no way out through TMA alone)
    const Plan pl = make_plan(T, N, K, swiglu, sm_count, c_by_tma && scale_part == nullptr && !emits, !swiglu && epilogue == 1);
    if (scale_part != nullptr || emits) {
        if (pl.persistent || pl.bn > 128) return CW_ERR_UNSUPPORTED;
        if (scale_part != nullptr && (scale_parts <= 0 || scale_dim <= 0)) return CW_ERR_BAD_SIZE;
        if (emits && (epilogue != 1 || swiglu || emit_g == nullptr || emit_part == nullptr)) return CW_ERR_UNSUPPORTED;
    }
    CUtensorMap mw, mw2, mx;
    if (make_map(&mw, W, N, K, K, BM) != 0) return CW_ERR_UNSUPPORTED;
    if (make_map(&mw2, swiglu ? W2 : W, N, K, K, BM) != 0) return CW_ERR_UNSUPPORTED;
    if (make_map(&mx, X, T, K, ldx, pl.pair ? pl.bn / 2 : pl.bn) != 0) return CW_ERR_UNSUPPORTED;
    const bool tma_store = (pl.splits == 1 || pl.pair) && c_by_tma && !emits;  // beginning a norm needs the new values in hand
    // prompt portions: the persistent kernel, whose epilogue overlaps the next tile's MMAs
    const bool persistent = pl.persistent;
    CUtensorMap mc = mx;
    if (tma_store && make_map_c(&mc, C, T, N, ldc, persistent ? P_CHUNK : pl.bn, c_f32) != 0) return CW_ERR_UNSUPPORTED;
    GemmParams p;
    p.tma_store = tma_store ? 1 : 0;
    p.T = T; p.N = N; p.K = K; p.ldc = ldc; p.epilogue = epilogue;
    p.num_kb = (K + BK - 1) / BK; p.kb_per_split = pl.kb_per_split; p.splits = pl.splits;
    p.bias = bias; p.C = C; p.status = status; p.bn = pl.bn;
    p.scale_part = scale_part; p.scale_parts = scale_parts; p.scale_eps = scale_eps; p.scale_dim = scale_dim;
    p.emit_g = emit_g; p.emit_x = (bf16*)emit_x; p.emit_part = emit_part;
    p.split_flags = g_split_flags;
    dim3 grid((N + BM - 1) / BM, (T + pl.bn - 1) / pl.bn, pl.splits);
    if (grid.y > 65535) return CW_ERR_BAD_SIZE;
    if (pl.pair) {
        const int units = pl.tiles * pl.splits;
        const int pairs = units < sm_count / 2 ? units : sm_count / 2;
        return swiglu ? launch_pair<true>(mw, mw2, mx, mc, p, pairs, stream) : launch_pair<false>(mw, mw2, mx, mc, p, pairs, stream);
    }
    if (persistent) {
        const int ctas = pl.tiles < sm_count ? pl.tiles : sm_count;
        if (pl.stream) return launch_persistent<64, false>(mw, mw2, mx, mc, p, ctas, stream);
        return swiglu ? launch_persistent<128, true>(mw, mw2, mx, mc, p, ctas, stream)
                      : launch_persistent<256, false>(mw, mw2, mx, mc, p, ctas, stream);
    }
#define CW_CASE(bn)                                                                       \
    case bn:                                                                              \
        return swiglu ? launch<bn, true>(mw, mw2, mx, mc, p, grid, stream)                \
                      : launch<bn, false>(mw, mw2, mx, mc, p, grid, stream);
    switch (pl.bn) {
        CW_CASE(16)
        CW_CASE(32)
        CW_CASE(64)
        CW_CASE(128)
        case 256:
            return launch<256, false>(mw, mw2, mx, mc, p, grid, stream);
    }
#undef CW_CASE
    return CW_ERR_UNSUPPORTED;
}

// How cw_gemm_tc_parts would split a product over K (1: not worth it, or too few tokens for the CTA-pair kernel).
extern "C" int cw_gemm_tc_parts_plan(int T, int N, int K, int sm_count, int* splits) {
    int bn = 0;
    *splits = 1;
    if (T <= 128 || T > PARTS_MAX_TOKENS || sm_count < 2 || !g_pair_enabled || T < g_persistent_from) return CW_OK;
    parts_plan(T, N, K, sm_count, splits, &bn);
    return CW_OK;
}

// parts[ks][t][n] = the part of X W^T that split ks of K contributes (float32, [splits][part_rows][N],
// part_rows >= T a multiple of 16; rows from T on are written too, with what the tile's last store
// holds).  `splits` as cw_gemm_tc_parts_plan gave it.
extern "C" int cw_gemm_tc_parts(const void* X, const void* W, float* parts, int T, int N, int K, int ldx, int part_rows,
                                int splits, int sm_count, int* status, cudaStream_t stream) {
    if (T == 0 || N == 0) return CW_OK;
    if (T < 0 || N < 0 || K <= 0 || ldx < K || part_rows < T || part_rows % P_CHUNK != 0) return CW_ERR_BAD_SIZE;
    if (K % 8 != 0 || ldx % 8 != 0 || N % 4 != 0 || ((uintptr_t)X & 15) || ((uintptr_t)W & 15) || ((uintptr_t)parts & 15))
        return CW_ERR_UNSUPPORTED;
    if (load_encode() != 0) return CW_ERR_UNSUPPORTED;
    int want = 1, bn = 0;
    if (T <= 128 || T > PARTS_MAX_TOKENS || sm_count < 2 || !g_pair_enabled || T < g_persistent_from) return CW_ERR_UNSUPPORTED;
    parts_plan(T, N, K, sm_count, &want, &bn);
    if (splits != want || splits < 1) return CW_ERR_BAD_SIZE;
    if (g_forced_bn != 0) bn = g_forced_bn;
    const int num_kb = (K + BK - 1) / BK;
    CUtensorMap mw, mx, mc;
    if (make_map(&mw, W, N, K, K, BM) != 0) return CW_ERR_UNSUPPORTED;
    if (make_map(&mx, X, T, K, ldx, bn / 2) != 0) return CW_ERR_UNSUPPORTED;
    if (make_map_c(&mc, parts, splits * part_rows, N, N, P_CHUNK, true) != 0) return CW_ERR_UNSUPPORTED;
    GemmParams p = {};
    p.tma_store = 1;
    p.T = T; p.N = N; p.K = K; p.ldc = N; p.epilogue = 3; p.part_rows = part_rows;
    p.num_kb = num_kb; p.kb_per_split = num_kb / splits; p.splits = splits;
    p.bias = nullptr; p.C = parts; p.status = status; p.bn = bn;
    p.split_flags = nullptr;
    const int tiles = ((N + 2 * BM - 1) / (2 * BM)) * ((T + bn - 1) / bn);
    const int units = tiles * splits;
    const int pairs = units < sm_count / 2 ? units : sm_count / 2;
    return launch_pair<false>(mw, mw, mx, mc, p, pairs, stream);
}

CW_TRACE_TU(gemm_tc)
