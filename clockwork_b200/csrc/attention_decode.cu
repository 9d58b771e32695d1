// Paged decode attention, the entry points (the kernel and how a step picks its variant: attention_decode_kernel.cuh).
#include "attention_decode_kernel.cuh"

// Workspace a call needs: part_o floats, part_lse floats, counters (one per (request, KV head, group of
// 16 query heads); with `two_levels`, one more per twelve splits of each, for the variant that merges
// many splits in two levels).
static void decode_workspace(int S, int nh, int nkv, int hd, int max_ctx, bool two_levels, long long* part_o_floats,
                             long long* part_lse_floats, int* counters) {
    const int splits = (max_ctx + MIN_SPLIT - 1) / MIN_SPLIT;
    const int G = nh / (nkv > 0 ? nkv : 1);
    *part_o_floats = (long long)S * nh * splits * hd;
    *part_lse_floats = (long long)S * nh * splits;
    *counters = S * nkv * ((G + 15) / 16) * (two_levels ? 1 + (splits + 11) / 12 : 1);
}

extern "C" int cw_attention_decode_workspace(int S, int nh, int nkv, int hd, int max_ctx, long long* part_o_floats,
                                             long long* part_lse_floats, int* counters) {
    decode_workspace(S, nh, nkv, hd, max_ctx, true, part_o_floats, part_lse_floats, counters);
    return CW_OK;
}

// q: [S, >= nh*hd] rows (row stride q_stride), one query token per request; out: [S, nh*hd].
// max_ctx bounds every ctx_lens[s]; it fixes the grid, not the result.  split (or *split_ptr): tokens
// per CTA, a multiple of 64 and at least 128; with split_ptr, split is 0 or an upper bound on *split_ptr
// (a smaller page list in shared memory: more CTAs per SM at long contexts).
extern "C" int cw_attention_decode_rows(const void* q, int q_stride, void* out, void* k_cache, void* v_cache,
                                        const int* block_tables, const int* ctx_lens, const int* q_start, int S, int nh,
                                        int nkv, int hd, int page_size, int max_blocks, int num_pages, float scale,
                                        int window, int max_ctx, int split, const int* split_ptr, float* part_o,
                                        float* part_lse, int* counters, int fuse_store, const float* inv_freq,
                                        int rotary_dim, const int* slots, int stages, int* status, cudaStream_t stream);

extern "C" int cw_attention_decode_fused(const void* q, int q_stride, void* out, void* k_cache, void* v_cache,
                                         const int* block_tables, const int* ctx_lens, int S, int nh, int nkv, int hd,
                                         int page_size, int max_blocks, int num_pages, float scale, int window,
                                         int max_ctx, int split, const int* split_ptr, float* part_o, float* part_lse,
                                         int* counters, int fuse_store, const float* inv_freq, int rotary_dim,
                                         const int* slots, int stages, int* status, cudaStream_t stream) {
    return cw_attention_decode_rows(q, q_stride, out, k_cache, v_cache, block_tables, ctx_lens, nullptr, S, nh, nkv, hd,
                                    page_size, max_blocks, num_pages, scale, window, max_ctx, split, split_ptr, part_o,
                                    part_lse, counters, fuse_store, inv_freq, rotary_dim, slots, stages, status, stream);
}

extern "C" int cw_attention_decode(const void* q, int q_stride, void* out, const void* k_cache, const void* v_cache,
                                   const int* block_tables, const int* ctx_lens, int S, int nh, int nkv, int hd,
                                   int page_size, int max_blocks, int num_pages, float scale, int window, int max_ctx,
                                   int split, const int* split_ptr, float* part_o, float* part_lse, int* counters, int* status, cudaStream_t stream) {
    return cw_attention_decode_fused(q, q_stride, out, const_cast<void*>(k_cache), const_cast<void*>(v_cache), block_tables,
                                     ctx_lens, S, nh, nkv, hd, page_size, max_blocks, num_pages, scale, window, max_ctx,
                                     split, split_ptr, part_o, part_lse, counters, 0, nullptr, 0, nullptr, 0, status, stream);
}

// As cw_attention_decode; with fuse_store != 0, q is the [q | k | v] row buffer that the QKV product
// wrote (raw): q and the new k are rotated here (inv_freq null: left alone) and the new token's k and
// v are stored at slots[s] before they are used, so no separate position/cache-write kernel runs.
// With q_start ([S + 1], may be null) the S requests are those of a flat batch that also holds prompt
// portions: request s owns rows q_start[s] .. q_start[s + 1] of q and out, and only the requests with
// exactly one row are served (the others are the prefill kernel's work); slots is then per row.
extern "C" int cw_attention_decode_rows(const void* q, int q_stride, void* out, void* k_cache, void* v_cache,
                                        const int* block_tables, const int* ctx_lens, const int* q_start, int S, int nh,
                                        int nkv, int hd, int page_size, int max_blocks, int num_pages, float scale,
                                        int window, int max_ctx, int split, const int* split_ptr, float* part_o,
                                        float* part_lse, int* counters, int fuse_store, const float* inv_freq,
                                        int rotary_dim, const int* slots, int stages, int* status, cudaStream_t stream) {
    if (S == 0) return CW_OK;
    if (S < 0 || nh <= 0 || nkv <= 0 || nh % nkv != 0 || page_size <= 0 || max_blocks <= 0 || max_ctx <= 0)
        return CW_ERR_BAD_SIZE;
    if (q_stride % 8 != 0 || ((uintptr_t)q & 15) || ((uintptr_t)k_cache & 15) || ((uintptr_t)v_cache & 15))
        return CW_ERR_UNSUPPORTED;
    if (S > 65535) return CW_ERR_BAD_SIZE;
    DecodeParams p;
    p.q = (const bf16*)q; p.q_stride = q_stride; p.out = (bf16*)out;
    p.k_cache = (const bf16*)k_cache; p.v_cache = (const bf16*)v_cache;
    p.block_tables = block_tables; p.ctx_lens = ctx_lens; p.q_start = q_start;
    p.nh = nh; p.nkv = nkv; p.qgroups = (nh / nkv + 15) / 16;
    p.page_size = page_size; p.page_shift = (page_size & (page_size - 1)) == 0 ? __builtin_ctz(page_size) : -1; p.max_blocks = max_blocks; p.num_pages = num_pages;
    p.scale = scale; p.window = window;
    p.part_o = part_o; p.part_lse = part_lse; p.counters = counters; p.status = status;
    if (fuse_store && (rotary_dim < 0 || rotary_dim > hd || (rotary_dim & 1))) return CW_ERR_BAD_SIZE;
    p.kv_new = fuse_store ? (const bf16*)q : nullptr;
    p.inv_freq = fuse_store ? inv_freq : nullptr;
    p.rotary_dim = fuse_store && inv_freq != nullptr ? rotary_dim : 0;
    p.slots = slots; p.k_cache_w = (bf16*)k_cache; p.v_cache_w = (bf16*)v_cache;
    p.num_slots = num_pages * page_size;
    p.stages = stages & 0xFF;        // tiles in flight
    p.swizzle = (stages >> 8) & 1;   // bit 8: the unpadded, swizzled K/V layout (with two tiles in flight)
    // bits 16..20: the splits of a group meet through a cluster of this many CTAs (2..16); 0: through the
    // workspace.  The grid's z extent is then the cluster and the kernel never cuts finer than it allows.
    p.cluster = (stages >> 16) & 0x1F;
    p.max_ctx = max_ctx;
    if (p.cluster > MAX_CLUSTER || hd > 128) p.cluster = 0;
    // bit 9: tiles by TMA, where the sizes allow it (else the variants above, with the same result)
    p.tma = ((stages >> 9) & 1) && hd % 64 == 0 && p.page_shift >= 3 && page_size <= TILE && !p.cluster && load_encode() == 0;
    // the grid is sized for the smallest split; a larger run-time split leaves the later CTAs idle
    if ((split_ptr == nullptr || split != 0) && (split < MIN_SPLIT || split % TILE != 0)) return CW_ERR_BAD_SIZE;
    int splits = (max_ctx + MIN_SPLIT - 1) / MIN_SPLIT;
    if (p.cluster > 1)
        splits = p.cluster;
    else
        p.cluster = 0;
    if (!p.cluster && splits > 1 && (part_o == nullptr || part_lse == nullptr || counters == nullptr)) return CW_ERR_BAD_SIZE;
    p.max_splits = splits;
    // few groups with contexts that can make more than 36 splits: the variant with the two-level merge
    p.tree = splits > 36 && S * nkv * p.qgroups <= 16 && !p.cluster && p.stages == 2;
    p.split = split; p.split_ptr = split_ptr;
    // when split_ptr decides at run time, `split` (if not 0) bounds what it may say, else a split may
    // span the whole context (a cluster makes the kernel cut no finer than the context bound divided
    // by its size); the bound sizes the page list in shared memory, and the kernel checks it
    const int least = p.cluster ? ((max_ctx + p.cluster - 1) / p.cluster + TILE - 1) / TILE * TILE : 0;
    const int host_split = split > least ? split : least;
    const int span = split_ptr != nullptr && split == 0 ? max_ctx : (host_split < max_ctx ? host_split : max_ctx);
    p.max_split_pages = (span + page_size - 1) / page_size + 1;
    if (splits > 65535) return CW_ERR_BAD_SIZE;
    switch (hd) {
        case 16: return launch_decode<16>(p, S, splits, stream);
        case 32: return launch_decode<32>(p, S, splits, stream);
        case 48: return launch_decode<48>(p, S, splits, stream);
        case 64: return launch_decode<64>(p, S, splits, stream);
        case 80:
        case 96:
        case 112:
        case 128: return cw_launch_decode_mid(hd, p, S, splits, stream);
        case 160:
        case 192:
        case 256: return cw_launch_decode_large(hd, p, S, splits, stream);
    }
    return CW_ERR_UNSUPPORTED;
}

// ---------------------------------------------------------------------------------------------
// The entry point that allocates nothing (declared and described in clockwork_b200.h).
// ---------------------------------------------------------------------------------------------
#include "clockwork_b200.h"

// Scratch of cw_attention_decode_noalloc: counters first, then the partial log-sum-exps, then the
// partial outputs.  Device code could name this array directly; host code cannot use the name as an
// address and asks the runtime for it once per device (below).
static __device__ __align__(256) unsigned char cw_noalloc_scratch[CW_NOALLOC_SCRATCH_BYTES];

#define CW_MAX_DEVICES 64
static void* g_noalloc_ptr[CW_MAX_DEVICES];  // device address of cw_noalloc_scratch, per device

static size_t align256(size_t n) { return (n + 255) & ~(size_t)255; }

extern "C" const char* cw_error_string(int code) {
    switch (code) {
        case CW_OK: return "success";
        case CW_ERR_BAD_SIZE: return "a size or stride argument is out of range";
        case CW_ERR_BAD_DTYPE: return "unknown dtype code";
        case CW_ERR_UNSUPPORTED: return "this combination of sizes or alignments is not supported";
        case CW_ERR_SETUP: return "set-up failed (no current device, or the scratch symbol could not be resolved)";
        case CW_ERR_SCRATCH_LIMIT: return "the call needs more scratch than the library's built-in CW_NOALLOC_SCRATCH_BYTES";
    }
    return code > 0 ? cudaGetErrorString((cudaError_t)code) : "unknown clockwork_b200 error code";
}

// The three parts of the scratch a call needs, each rounded up to 256 bytes.
static void noalloc_layout(int S, int nh, int nkv, int hd, int max_ctx, size_t* counters_bytes, size_t* lse_bytes,
                           size_t* o_bytes) {
    long long part_o_floats = 0, part_lse_floats = 0;
    int counters = 0;
    // (this entry point asks for four tiles in flight: never the variant with the two-level merge)
    decode_workspace(S, nh, nkv, hd, max_ctx, false, &part_o_floats, &part_lse_floats, &counters);
    *counters_bytes = align256((size_t)counters * sizeof(int));
    *lse_bytes = align256((size_t)part_lse_floats * sizeof(float));
    *o_bytes = align256((size_t)part_o_floats * sizeof(float));
}

extern "C" int cw_attention_decode_noalloc_fits(int S, int nh, int nkv, int hd, int max_ctx) {
    if (S < 0 || nh <= 0 || nkv <= 0 || nh % nkv != 0 || hd <= 0 || max_ctx <= 0) return CW_ERR_BAD_SIZE;
    if (S == 0) return 1;
    size_t counters_bytes, lse_bytes, o_bytes;
    noalloc_layout(S, nh, nkv, hd, max_ctx, &counters_bytes, &lse_bytes, &o_bytes);
    return counters_bytes + lse_bytes + o_bytes <= (size_t)CW_NOALLOC_SCRATCH_BYTES ? 1 : 0;
}

extern "C" int cw_attention_decode_noalloc(const void* q, int q_stride, void* out, const void* k_cache,
                                           const void* v_cache, const int* block_tables, const int* ctx_lens, int S,
                                           int nh, int nkv, int hd, int page_size, int max_blocks, int num_pages,
                                           float scale, int window, int max_ctx, int split, int* status,
                                           cudaStream_t stream) {
    if (S == 0) return CW_OK;
    if (S < 0 || nh <= 0 || nkv <= 0 || nh % nkv != 0 || hd <= 0 || max_ctx <= 0) return CW_ERR_BAD_SIZE;
    size_t counters_bytes, lse_bytes, o_bytes;
    noalloc_layout(S, nh, nkv, hd, max_ctx, &counters_bytes, &lse_bytes, &o_bytes);
    if (counters_bytes + lse_bytes + o_bytes > (size_t)CW_NOALLOC_SCRATCH_BYTES) return CW_ERR_SCRATCH_LIMIT;

    // once per device, with that device current: the array's device address
    int device = -1;
    if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= CW_MAX_DEVICES) return CW_ERR_SETUP;
    if (g_noalloc_ptr[device] == nullptr) {
        void* ptr = nullptr;
        const cudaError_t err = cudaGetSymbolAddress(&ptr, cw_noalloc_scratch);
        if (err != cudaSuccess || ptr == nullptr) return err != cudaSuccess ? (int)err : CW_ERR_SETUP;
        g_noalloc_ptr[device] = ptr;
    }
    unsigned char* base = (unsigned char*)g_noalloc_ptr[device];
    // the array keeps the last call's contents: the counters must start at zero
    const cudaError_t err = cudaMemsetAsync(base, 0, counters_bytes, stream);
    if (err != cudaSuccess) return (int)err;
    return cw_attention_decode(q, q_stride, out, k_cache, v_cache, block_tables, ctx_lens, S, nh, nkv, hd, page_size,
                               max_blocks, num_pages, scale, window, max_ctx, split, nullptr,
                               (float*)(base + counters_bytes + lse_bytes), (float*)(base + counters_bytes),
                               (int*)base, status, stream);
}

CW_TRACE_TU(attention_decode)
