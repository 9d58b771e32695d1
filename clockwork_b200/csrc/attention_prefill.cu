// Paged causal attention for prompt portions in bfloat16 (flash-attention style): a CTA owns 128
// query tokens of one request and one query head, streams the request's keys and values from the
// cache in tiles of 64 tokens (through the block table), and keeps scores, softmax statistics and
// the output accumulator in registers.  QK^T and P.V run on the tensor cores (mma.sync m16n8k16),
// softmax in float32; probabilities are rounded to bfloat16 for P.V.
//
// Reference: clockwork/kernels/attention.py:68-96 (gather the context through one block table, then
// dense causal attention with the query aligned to the end of the context, :45-65) and
// clockwork/engine/model.py:103-118 (one call per sequence of the batch).  Here one launch covers
// every portion of the batch: the host lists (request, first query row) work items, one per 128 query
// tokens.  A decoded token is a portion of length one and may ride along.
#include "attention_mma.cuh"

#define QT 128   // query rows per CTA (16 per warp)
#define TILE 64  // keys per staged tile
#define NWARPS 8

struct PrefillParams {
    const bf16* q; int q_stride;
    bf16* out;
    const bf16* k_cache; const bf16* v_cache;
    const int* block_tables; const int* q_start; const int* ctx_lens;
    const int* item_seq; const int* item_q0;
    int nh, nkv, page_size, page_shift, max_blocks, num_pages;
    float scale; int window;
    int* status;
};

template <int HD>
__global__ void __launch_bounds__(NWARPS * 32)
attn_prefill_kernel(const PrefillParams p) {
    constexpr int LD = HD + 8;
    extern __shared__ __align__(16) uint8_t smem_raw[];
    bf16* Qs = (bf16*)smem_raw;      // [QT][LD]
    bf16* Ks = Qs + QT * LD;         // [2][TILE][LD]
    bf16* Vs = Ks + 2 * TILE * LD;   // [2][TILE][LD]

    pdl_launch_dependents();
    pdl_wait();
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, t = lane & 3;
    const int s = p.item_seq[blockIdx.x], q0 = p.item_q0[blockIdx.x];
    if (s < 0) return;  // an unused entry of a work list of fixed length (captured steps)
    const int h = blockIdx.y, kvh = h / (p.nh / p.nkv);
    const int row0 = p.q_start[s], q_len = p.q_start[s + 1] - row0;
    const int ctx = p.ctx_lens[s];
    const int pos0 = ctx - q_len + q0;              // position of the tile's first query
    const int nq = min(QT, q_len - q0);             // query rows in this tile
    const int kv_hi = pos0 + nq;                    // keys [.., kv_hi) are visible to the last row
    const int kv_lo = p.window > 0 ? max(0, pos0 + 1 - p.window) : 0;
    const int tile_lo = kv_lo / TILE * TILE;
    const int* table = p.block_tables + (size_t)s * p.max_blocks;
    const float scale_log2 = p.scale * 1.4426950408889634f;  // softmax in base 2: exp(x) = 2^(x log2 e)

    for (int i = tid; i < QT * (HD / 8); i += blockDim.x) {
        const int r = i / (HD / 8), c = i % (HD / 8);
        uint4 v = make_uint4(0, 0, 0, 0);
        if (r < nq) v = *reinterpret_cast<const uint4*>(p.q + (size_t)(row0 + q0 + r) * p.q_stride + (size_t)h * HD + c * 8);
        *reinterpret_cast<uint4*>(Qs + r * LD + c * 8) = v;
    }

    // Every thread copies the same 16-byte column of several rows: the row's cache slot is worked
    // out once per row and the rest of the addressing is compile-time strides.
    constexpr int CH = HD / 8;
    constexpr bool EVEN = (NWARPS * 32) % CH == 0;
    constexpr int RPP = EVEN ? (NWARPS * 32) / CH : 1;
    auto slot_of = [&](int pos) -> int {
        if (pos >= kv_hi || pos < kv_lo) return -1;
        const int blk = p.page_shift >= 0 ? pos >> p.page_shift : pos / p.page_size;
        const int page = blk < p.max_blocks ? table[blk] : -1;
        if (page < 0 || page >= p.num_pages) {
            cw_report(p.status, CW_ST_PAGE_RANGE, s, page);
            return -1;
        }
        return page * p.page_size + (p.page_shift >= 0 ? pos & (p.page_size - 1) : pos % p.page_size);
    };
    auto copy_chunk = [&](bf16* kd, bf16* vd, int r, int c, int slot) {
        if (slot >= 0) {
            const size_t src = ((size_t)slot * p.nkv + kvh) * HD + c * 8;
            cp_async16(kd + r * LD + c * 8, p.k_cache + src);
            cp_async16(vd + r * LD + c * 8, p.v_cache + src);
        } else {
            *reinterpret_cast<uint4*>(kd + r * LD + c * 8) = make_uint4(0, 0, 0, 0);
            *reinterpret_cast<uint4*>(vd + r * LD + c * 8) = make_uint4(0, 0, 0, 0);
        }
    };
    auto load_tile = [&](int tile0, int buf) {
        bf16* kd = Ks + buf * TILE * LD;
        bf16* vd = Vs + buf * TILE * LD;
        if (EVEN) {
            const int c = tid % CH, r0 = tid / CH;
#pragma unroll
            for (int k = 0; k < (TILE + RPP - 1) / RPP; ++k) {
                const int r = r0 + k * RPP;
                if (r < TILE) copy_chunk(kd, vd, r, c, slot_of(tile0 + r));
            }
        } else {
            for (int i = tid; i < TILE * CH; i += blockDim.x) copy_chunk(kd, vd, i / CH, i % CH, slot_of(tile0 + i / CH));
        }
        cp_async_commit();
    };

    const int ntiles = (kv_hi - tile_lo + TILE - 1) / TILE;
    load_tile(tile_lo, 0);
    __syncthreads();

    float o_acc[HD / 8][4];
#pragma unroll
    for (int i = 0; i < HD / 8; ++i) o_acc[i][0] = o_acc[i][1] = o_acc[i][2] = o_acc[i][3] = 0.f;
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
    const int qrow = warp * 16;                    // this warp's first query row within the tile
    const int qpos[2] = {pos0 + qrow + g, pos0 + qrow + g + 8};
    const bool warp_active = qrow < nq;

    for (int it = 0; it < ntiles; ++it) {
        const int buf = it & 1;
        const int tile0 = tile_lo + it * TILE;
        if (it + 1 < ntiles) {
            load_tile(tile0 + TILE, buf ^ 1);
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncthreads();
        // a warp skips tiles that lie wholly after its last query or wholly before its first window
        const int w_last = pos0 + min(qrow + 15, nq - 1);
        const int w_first_lo = p.window > 0 ? pos0 + qrow + 1 - p.window : 0;
        if (warp_active && tile0 <= w_last && tile0 + TILE > w_first_lo) {
            const bf16* kt = Ks + buf * TILE * LD;
            const bf16* vt = Vs + buf * TILE * LD;
            float sc[TILE / 8][4];
#pragma unroll
            for (int j = 0; j < TILE / 8; ++j) sc[j][0] = sc[j][1] = sc[j][2] = sc[j][3] = 0.f;
#pragma unroll
            for (int ks = 0; ks < HD / 16; ++ks) {
                uint32_t qa[4];
                ldmatrix_x4(smem_addr(Qs + (qrow + (lane & 7) + 8 * ((lane >> 3) & 1)) * LD + ks * 16 + 8 * (lane >> 4)),
                            qa[0], qa[1], qa[2], qa[3]);
#pragma unroll
                for (int j2 = 0; j2 < TILE / 16; ++j2) {
                    uint32_t b0, b1, b2, b3;
                    ldmatrix_x4(smem_addr(kt + (j2 * 16 + (lane & 7) + 8 * (lane >> 4)) * LD + ks * 16 + 8 * ((lane >> 3) & 1)),
                                b0, b1, b2, b3);
                    mma_bf16(sc[2 * j2], qa, b0, b1);
                    mma_bf16(sc[2 * j2 + 1], qa, b2, b3);
                }
            }
            // only tiles that touch the diagonal, the window's lower edge or the context's end need
            // the per-element test; the others are wholly visible to all 16 rows of the warp
            const int w_first = pos0 + qrow;
            const bool all_visible = tile0 + TILE - 1 <= w_first && tile0 >= kv_lo &&
                                     (p.window <= 0 || tile0 > w_last - p.window);
            float mx[2] = {-INFINITY, -INFINITY};
            if (all_visible) {
#pragma unroll
                for (int j = 0; j < TILE / 8; ++j)
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        sc[j][e] *= scale_log2;
                        mx[e >> 1] = fmaxf(mx[e >> 1], sc[j][e]);
                    }
            } else {
#pragma unroll
                for (int j = 0; j < TILE / 8; ++j)
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const int pos = tile0 + 8 * j + 2 * t + (e & 1);
                        const int qp = qpos[e >> 1];
                        const bool vis = pos <= qp && pos >= kv_lo && (p.window <= 0 || pos > qp - p.window);
                        const float v = vis ? sc[j][e] * scale_log2 : -INFINITY;
                        sc[j][e] = v;
                        mx[e >> 1] = fmaxf(mx[e >> 1], v);
                    }
            }
            float alpha[2];
#pragma unroll
            for (int r = 0; r < 2; ++r) {
                mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
                mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
                const float m_new = fmaxf(m_run[r], mx[r]);
                alpha[r] = (m_run[r] == -INFINITY) ? 0.f : fast_exp2(m_run[r] - m_new);
                float sum = 0.f;
#pragma unroll
                for (int j = 0; j < TILE / 8; ++j)
#pragma unroll
                    for (int e = 0; e < 2; ++e) {
                        const float pr = (m_new == -INFINITY) ? 0.f : fast_exp2(sc[j][2 * r + e] - m_new);
                        sc[j][2 * r + e] = pr;
                        sum += pr;
                    }
                l_run[r] = l_run[r] * alpha[r] + sum;
                m_run[r] = m_new;
            }
#pragma unroll
            for (int i = 0; i < HD / 8; ++i) {
                o_acc[i][0] *= alpha[0]; o_acc[i][1] *= alpha[0];
                o_acc[i][2] *= alpha[1]; o_acc[i][3] *= alpha[1];
            }
#pragma unroll
            for (int kk = 0; kk < TILE / 16; ++kk) {
                uint32_t pa[4];
                pa[0] = pack_bf16(sc[2 * kk][0], sc[2 * kk][1]);
                pa[1] = pack_bf16(sc[2 * kk][2], sc[2 * kk][3]);
                pa[2] = pack_bf16(sc[2 * kk + 1][0], sc[2 * kk + 1][1]);
                pa[3] = pack_bf16(sc[2 * kk + 1][2], sc[2 * kk + 1][3]);
#pragma unroll
                for (int n2 = 0; n2 < HD / 16; ++n2) {
                    uint32_t v0, v1, v2, v3;
                    ldmatrix_x4_trans(smem_addr(vt + (kk * 16 + (lane & 7) + 8 * ((lane >> 3) & 1)) * LD + n2 * 16 + 8 * (lane >> 4)),
                                      v0, v1, v2, v3);
                    mma_bf16(o_acc[2 * n2], pa, v0, v1);
                    mma_bf16(o_acc[2 * n2 + 1], pa, v2, v3);
                }
            }
        }
        __syncthreads();
    }
    if (!warp_active) return;
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 1);
        l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 2);
    }
    const float inv[2] = {l_run[0] > 0.f ? 1.f / l_run[0] : 0.f, l_run[1] > 0.f ? 1.f / l_run[1] : 0.f};
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const int qr = qrow + g + 8 * r;
        if (qr >= nq) continue;
        bf16* o = p.out + ((size_t)(row0 + q0 + qr) * p.nh + h) * HD;
#pragma unroll
        for (int nt = 0; nt < HD / 8; ++nt) {
            const uint32_t v = pack_bf16(o_acc[nt][2 * r] * inv[r], o_acc[nt][2 * r + 1] * inv[r]);
            *reinterpret_cast<uint32_t*>(o + nt * 8 + 2 * t) = v;
        }
    }
}

template <int HD>
static int launch_prefill(const PrefillParams& p, int items, cudaStream_t stream) {
    constexpr int LD = HD + 8;
    constexpr int SMEM = (QT * LD + 4 * TILE * LD) * 2;
    static bool configured = false;
    if (!configured) {
        if (SMEM > 48 * 1024 &&
            cudaFuncSetAttribute(attn_prefill_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM) != cudaSuccess)
            return (int)cudaGetLastError();
        configured = true;
    }
    dim3 grid(items, p.nh);
    return cw_launch(attn_prefill_kernel<HD>, grid, dim3(NWARPS * 32), SMEM, stream, 1, p);
}

// q: [N, >= nh*hd] rows of the flat batch; out: [N, nh*hd]; item_seq/item_q0: one entry per 128
// query rows of each request (request index within the step, first query row within its portion).
extern "C" int cw_attention_prefill(const void* q, int q_stride, void* out, const void* k_cache, const void* v_cache,
                                    const int* block_tables, const int* q_start, const int* ctx_lens,
                                    const int* item_seq, const int* item_q0, int items, int nh, int nkv, int hd,
                                    int page_size, int max_blocks, int num_pages, float scale, int window,
                                    int* status, cudaStream_t stream) {
    if (items == 0) return CW_OK;
    if (items < 0 || nh <= 0 || nkv <= 0 || nh % nkv != 0 || page_size <= 0 || max_blocks <= 0) return CW_ERR_BAD_SIZE;
    if (q_stride % 8 != 0 || ((uintptr_t)q & 15) || ((uintptr_t)k_cache & 15) || ((uintptr_t)v_cache & 15))
        return CW_ERR_UNSUPPORTED;
    if (nh > 65535) return CW_ERR_BAD_SIZE;
    PrefillParams p;
    p.q = (const bf16*)q; p.q_stride = q_stride; p.out = (bf16*)out;
    p.k_cache = (const bf16*)k_cache; p.v_cache = (const bf16*)v_cache;
    p.block_tables = block_tables; p.q_start = q_start; p.ctx_lens = ctx_lens;
    p.item_seq = item_seq; p.item_q0 = item_q0;
    p.nh = nh; p.nkv = nkv; p.page_size = page_size; p.page_shift = (page_size & (page_size - 1)) == 0 ? __builtin_ctz(page_size) : -1; p.max_blocks = max_blocks; p.num_pages = num_pages;
    p.scale = scale; p.window = window; p.status = status;
    switch (hd) {
        case 16: return launch_prefill<16>(p, items, stream);
        case 32: return launch_prefill<32>(p, items, stream);
        case 48: return launch_prefill<48>(p, items, stream);
        case 64: return launch_prefill<64>(p, items, stream);
        case 80: return launch_prefill<80>(p, items, stream);
        case 96: return launch_prefill<96>(p, items, stream);
        case 112: return launch_prefill<112>(p, items, stream);
        case 128: return launch_prefill<128>(p, items, stream);
    }
    return CW_ERR_UNSUPPORTED;
}

CW_TRACE_TU(attention_prefill)
