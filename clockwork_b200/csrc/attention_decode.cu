// Paged decode attention in bfloat16: every request brings one query token and reads its whole
// context from the cache.  The step is a stream of K/V pages from HBM, so the context of a request
// is split over CTAs (256 tokens each) and all query heads of one KV head share each K/V tile.
//
// Reference: clockwork/kernels/attention.py:113-134 (masking keys >= ctx_len, softmax, P.V) and the
// Triton kernel clockwork/kernels/triton_paged_attn.py:16-106 (online softmax over one page per
// iteration, float32 accumulation).  That kernel runs one program per (sequence, query head), so
// every query head re-reads its KV head (:49); here a CTA is (KV head, sequence, context split), the
// group's query heads are the 16 rows of a tensor-core tile (mma.sync m16n8k16), and the splits are
// merged by the CTA that finishes last, in split order.
//
// Scores, softmax and accumulation are float32; probabilities are rounded to bfloat16 for P.V.
#include "attention_mma.cuh"

#define TILE 64
#define SPLIT 256
#define NWARPS 4

struct DecodeParams {
    const bf16* q; int q_stride;
    bf16* out;
    const bf16* k_cache; const bf16* v_cache;
    const int* block_tables; const int* ctx_lens;
    int nh, nkv, qgroups, page_size, page_shift, max_blocks, num_pages;
    float scale; int window;
    float* part_o;   // [S, nh, max_splits, HD]
    float* part_lse; // [S, nh, max_splits]
    int max_splits;
    int* counters;   // [S * nkv * qgroups]
    int* status;
};

__device__ __forceinline__ void cp_async_wait_upto(int n) {
    switch (n) {
        case 0: cp_async_wait<0>(); break;
        case 1: cp_async_wait<1>(); break;
        case 2: cp_async_wait<2>(); break;
        default: cp_async_wait<3>(); break;
    }
}

// ST: tiles in flight.  4 puts a whole split (256 tokens) in flight at once, for steps with few
// CTAs where latency is everything; 2 halves the shared memory so that two CTAs share an SM.
template <int HD, int ST>
__global__ void __launch_bounds__(NWARPS * 32)
attn_decode_kernel(const DecodeParams p) {
    constexpr int LD = HD + 8;  // padded row (elements): consecutive rows fall into different banks
    extern __shared__ __align__(16) uint8_t smem_raw[];
    bf16* Qs = (bf16*)smem_raw;                 // [16][LD]
    bf16* Ks = Qs + 16 * LD;                    // [ST][TILE][LD]
    bf16* Vs = Ks + ST * TILE * LD;             // [ST][TILE][LD]
    __shared__ float ml_s[NWARPS][16][2];
    __shared__ int slot_s[SPLIT];               // cache slot of every token of this split (-1: none)
    __shared__ int last_flag;

    pdl_launch_dependents();
    pdl_wait();
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, t = lane & 3;
    const int kvh = blockIdx.x / p.qgroups, qg = blockIdx.x % p.qgroups;
    const int s = blockIdx.y, sp = blockIdx.z;
    const int G = p.nh / p.nkv;
    const int h0 = kvh * G + qg * 16;
    const int rows = min(16, G - qg * 16);
    const int ctx = p.ctx_lens[s];
    if (ctx <= 0) {  // a padding row of a fixed-shape batch
        if (sp == 0)
            for (int i = tid; i < rows * HD; i += blockDim.x)
                p.out[((size_t)s * p.nh + h0 + i / HD) * HD + i % HD] = __float2bfloat16_rn(0.f);
        return;
    }
    const int kv_begin = p.window > 0 ? max(0, ctx - p.window) : 0;
    const int nsplits = (ctx + SPLIT - 1) / SPLIT;
    const int first_split = kv_begin / SPLIT;
    if (sp < first_split || sp >= nsplits) return;
    const int t0 = sp * SPLIT, t1 = min(ctx, t0 + SPLIT);
    const int* table = p.block_tables + (size_t)s * p.max_blocks;
    const float scale_log2 = p.scale * 1.4426950408889634f;  // softmax in base 2: exp(x) = 2^(x log2 e)

    // ---- Q rows of this group into shared memory, then into A fragments ----------------------------
    for (int i = tid; i < 16 * (HD / 8); i += blockDim.x) {
        const int r = i / (HD / 8), c = i % (HD / 8);
        uint4 v = make_uint4(0, 0, 0, 0);
        if (r < rows) v = *reinterpret_cast<const uint4*>(p.q + (size_t)s * p.q_stride + (size_t)(h0 + r) * HD + c * 8);
        *reinterpret_cast<uint4*>(Qs + r * LD + c * 8) = v;
    }

    // slots of the split's tokens, looked up once: tile loads then depend on shared memory only
    for (int i = tid; i < SPLIT; i += blockDim.x) {
        const int pos = t0 + i;
        int slot = -1;
        if (pos < t1 && pos >= kv_begin) {
            const int blk = p.page_shift >= 0 ? pos >> p.page_shift : pos / p.page_size;
            const int page = blk < p.max_blocks ? table[blk] : -1;
            if (page < 0 || page >= p.num_pages) {
                cw_report(p.status, CW_ST_PAGE_RANGE, s, page);
            } else {
                slot = page * p.page_size + (p.page_shift >= 0 ? pos & (p.page_size - 1) : pos % p.page_size);
            }
        }
        slot_s[i] = slot;
    }
    __syncthreads();  // Qs and slot_s visible

    auto load_tile = [&](int tile_idx) {
        bf16* kd = Ks + (tile_idx % ST) * TILE * LD;
        bf16* vd = Vs + (tile_idx % ST) * TILE * LD;
        for (int i = tid; i < TILE * (HD / 8); i += blockDim.x) {
            const int r = i / (HD / 8), c = i % (HD / 8);
            const int slot = slot_s[tile_idx * TILE + r];
            if (slot >= 0) {
                const size_t src = ((size_t)slot * p.nkv + kvh) * HD + c * 8;
                cp_async16(kd + r * LD + c * 8, p.k_cache + src);
                cp_async16(vd + r * LD + c * 8, p.v_cache + src);
            } else {
                *reinterpret_cast<uint4*>(kd + r * LD + c * 8) = make_uint4(0, 0, 0, 0);
                *reinterpret_cast<uint4*>(vd + r * LD + c * 8) = make_uint4(0, 0, 0, 0);
            }
        }
        cp_async_commit();
    };

    const int ntiles = (t1 - t0 + TILE - 1) / TILE;
    for (int i = 0; i < ST && i < ntiles; ++i) load_tile(i);
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
        cp_async_wait_upto(min(ntiles - it - 1, ST - 1));  // tile `it` has landed; later ones may fly
        __syncthreads();
        const bf16* kt = Ks + buf * TILE * LD + warp * 16 * LD;
        const bf16* vt = Vs + buf * TILE * LD + warp * 16 * LD;
        const int tok0 = t0 + it * TILE + warp * 16;  // first token of this warp's 16
        if (tok0 < t1) {
            float sc[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll
            for (int ks = 0; ks < HD / 16; ++ks) {
                uint32_t b0, b1, b2, b3;
                ldmatrix_x4(smem_addr(kt + ((lane & 7) + 8 * (lane >> 4)) * LD + ks * 16 + 8 * ((lane >> 3) & 1)),
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
                alpha[r] = (m_run[r] == -INFINITY) ? 0.f : exp2f(m_run[r] - m_new);
                float sum = 0.f;
#pragma unroll
                for (int j = 0; j < 2; ++j)
#pragma unroll
                    for (int e = 0; e < 2; ++e) {
                        const float v = sc[j][2 * r + e];
                        const float pr = (m_new == -INFINITY) ? 0.f : exp2f(v - m_new);
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
                ldmatrix_x4_trans(smem_addr(vt + ((lane & 7) + 8 * ((lane >> 3) & 1)) * LD + n2 * 16 + 8 * (lane >> 4)),
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
    const int active = nsplits - first_split;
    for (int i = tid; i < rows * HD; i += blockDim.x) {
        const int r = i / HD, d = i % HD;
        float m = -INFINITY;
#pragma unroll
        for (int w = 0; w < NWARPS; ++w) m = fmaxf(m, ml_s[w][r][0]);
        float L = 0.f, O = 0.f;
        if (m != -INFINITY) {
#pragma unroll
            for (int w = 0; w < NWARPS; ++w) {
                const float mw = ml_s[w][r][0];
                const float e = (mw == -INFINITY) ? 0.f : exp2f(mw - m);
                L += e * ml_s[w][r][1];
                O += e * Om[((size_t)w * 16 + r) * HD + d];
            }
        }
        const float val = L > 0.f ? O / L : 0.f;
        const int h = h0 + r;
        if (active == 1) {
            p.out[((size_t)s * p.nh + h) * HD + d] = __float2bfloat16_rn(val);
        } else {
            p.part_o[(((size_t)s * p.nh + h) * p.max_splits + sp) * HD + d] = val;
            if (d == 0) p.part_lse[((size_t)s * p.nh + h) * p.max_splits + sp] = L > 0.f ? m + log2f(L) : -INFINITY;  // base 2
        }
    }
    if (active == 1) return;
    // ---- the CTA that finishes last merges the splits, in split order ------------------------------
    __threadfence();
    __syncthreads();
    if (tid == 0) {
        int* counter = p.counters + ((size_t)s * p.nkv + kvh) * p.qgroups + qg;
        const int prev = atomicAdd(counter, 1);
        last_flag = (prev == active - 1);
        if (last_flag) *counter = 0;
    }
    __syncthreads();
    if (!last_flag) return;
    __threadfence();
    for (int i = tid; i < rows * HD; i += blockDim.x) {
        const int r = i / HD, d = i % HD, h = h0 + r;
        const float* lse = p.part_lse + ((size_t)s * p.nh + h) * p.max_splits;
        const float* po = p.part_o + ((size_t)s * p.nh + h) * p.max_splits * HD + d;
        float m = -INFINITY;
        for (int k0 = first_split; k0 < nsplits; k0 += 8) {  // eight independent loads at a time
            float l8[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) l8[j] = (k0 + j < nsplits) ? __ldcg(lse + k0 + j) : -INFINITY;
#pragma unroll
            for (int j = 0; j < 8; ++j) m = fmaxf(m, l8[j]);
        }
        float W = 0.f, O = 0.f;
        if (m != -INFINITY)
            for (int k0 = first_split; k0 < nsplits; k0 += 8) {
                float l8[8], o8[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const bool in = k0 + j < nsplits;
                    l8[j] = in ? __ldcg(lse + k0 + j) : -INFINITY;
                    o8[j] = in ? __ldcg(po + (size_t)(k0 + j) * HD) : 0.f;
                }
#pragma unroll
                for (int j = 0; j < 8; ++j) {  // split order
                    const float e = (l8[j] == -INFINITY) ? 0.f : exp2f(l8[j] - m);
                    W += e;
                    O += e * o8[j];
                }
            }
        p.out[((size_t)s * p.nh + h) * HD + d] = __float2bfloat16_rn(W > 0.f ? O / W : 0.f);
    }
}

template <int HD, int ST>
static int launch_decode_st(const DecodeParams& p, int S, int splits, cudaStream_t stream) {
    constexpr int LD = HD + 8;
    constexpr int SMEM = (16 * LD + 2 * ST * TILE * LD) * 2;
    constexpr int MERGE = NWARPS * 16 * HD * 4;
    static_assert(MERGE <= ST * TILE * LD * 2, "the merge buffer must fit over the K buffers");
    static bool configured = false;
    if (!configured) {
        if (SMEM > 48 * 1024 &&
            cudaFuncSetAttribute(attn_decode_kernel<HD, ST>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM) != cudaSuccess)
            return (int)cudaGetLastError();
        configured = true;
    }
    dim3 grid(p.nkv * p.qgroups, S, splits);
    return cw_launch(attn_decode_kernel<HD, ST>, grid, dim3(NWARPS * 32), SMEM, stream, 1, p);
}

template <int HD>
static int launch_decode(const DecodeParams& p, int S, int splits, cudaStream_t stream) {
    // few CTAs: a whole split in flight per CTA; many CTAs: two CTAs per SM instead
    const long long ctas = (long long)p.nkv * p.qgroups * S * splits;
    if (HD <= 128 && ctas <= 2 * 148) return launch_decode_st<HD, (HD <= 128 ? 4 : 2)>(p, S, splits, stream);
    return launch_decode_st<HD, 2>(p, S, splits, stream);
}

// Workspace a call needs: part_o floats, part_lse floats, counters.
extern "C" int cw_attention_decode_workspace(int S, int nh, int nkv, int hd, int max_ctx, long long* part_o_floats,
                                             long long* part_lse_floats, int* counters) {
    const int splits = (max_ctx + SPLIT - 1) / SPLIT;
    const int G = nh / (nkv > 0 ? nkv : 1);
    *part_o_floats = (long long)S * nh * splits * hd;
    *part_lse_floats = (long long)S * nh * splits;
    *counters = S * nkv * ((G + 15) / 16);
    return CW_OK;
}

// q: [S, >= nh*hd] rows (row stride q_stride), one query token per request; out: [S, nh*hd].
// max_ctx bounds every ctx_lens[s]; it fixes the grid, not the result.
extern "C" int cw_attention_decode(const void* q, int q_stride, void* out, const void* k_cache, const void* v_cache,
                                   const int* block_tables, const int* ctx_lens, int S, int nh, int nkv, int hd,
                                   int page_size, int max_blocks, int num_pages, float scale, int window, int max_ctx,
                                   float* part_o, float* part_lse, int* counters, int* status, cudaStream_t stream) {
    if (S == 0) return CW_OK;
    if (S < 0 || nh <= 0 || nkv <= 0 || nh % nkv != 0 || page_size <= 0 || max_blocks <= 0 || max_ctx <= 0)
        return CW_ERR_BAD_SIZE;
    if (q_stride % 8 != 0 || ((uintptr_t)q & 15) || ((uintptr_t)k_cache & 15) || ((uintptr_t)v_cache & 15))
        return CW_ERR_UNSUPPORTED;
    if (S > 65535) return CW_ERR_BAD_SIZE;
    DecodeParams p;
    p.q = (const bf16*)q; p.q_stride = q_stride; p.out = (bf16*)out;
    p.k_cache = (const bf16*)k_cache; p.v_cache = (const bf16*)v_cache;
    p.block_tables = block_tables; p.ctx_lens = ctx_lens;
    p.nh = nh; p.nkv = nkv; p.qgroups = (nh / nkv + 15) / 16;
    p.page_size = page_size; p.page_shift = (page_size & (page_size - 1)) == 0 ? __builtin_ctz(page_size) : -1; p.max_blocks = max_blocks; p.num_pages = num_pages;
    p.scale = scale; p.window = window;
    p.part_o = part_o; p.part_lse = part_lse; p.counters = counters; p.status = status;
    const int splits = (max_ctx + SPLIT - 1) / SPLIT;
    p.max_splits = splits;
    if (splits > 65535) return CW_ERR_BAD_SIZE;
    switch (hd) {
        case 16: return launch_decode<16>(p, S, splits, stream);
        case 32: return launch_decode<32>(p, S, splits, stream);
        case 48: return launch_decode<48>(p, S, splits, stream);
        case 64: return launch_decode<64>(p, S, splits, stream);
        case 80: return launch_decode<80>(p, S, splits, stream);
        case 96: return launch_decode<96>(p, S, splits, stream);
        case 112: return launch_decode<112>(p, S, splits, stream);
        case 128: return launch_decode<128>(p, S, splits, stream);
        case 160: return launch_decode<160>(p, S, splits, stream);
        case 192: return launch_decode<192>(p, S, splits, stream);
        case 256: return launch_decode<256>(p, S, splits, stream);
    }
    return CW_ERR_UNSUPPORTED;
}
