// Paged causal attention, general form: any mixture of prompt portions and single decoded
// tokens, any head count / group size / head size, optional window.  One thread block per
// (token, query head); float32 scores, softmax and accumulation in both run precisions.
//
// Reference: clockwork/kernels/attention.py:45-65 (scores = q.k * scale with the scale applied
// after the dot product, key j visible to the query at absolute position p iff j <= p,
// softmax, P.V), :35-42 (query head h reads KV head h // (nh/nkv)), :68-96 and :113-134 (keys
// and values gathered through the request's block table).  A token's keys are those of its own
// request at positions [max(0, p+1-window), p]; they are read from the cache, where this step's
// tokens were written before (clockwork/engine/model.py:100-127).
//
// Keys are processed in chunks of 128 starting at the first visible key; the chunking depends
// on the token's position and the window only, never on the rest of the batch.
#include "common.cuh"

#define CH 128

template <typename T>
__global__ void __launch_bounds__(CH)
attn_ref_kernel(const T* __restrict__ q, int q_stride, T* __restrict__ out,
                const T* __restrict__ k_cache, const T* __restrict__ v_cache,
                const int* __restrict__ block_tables, const int* __restrict__ tok_seq,
                const int* __restrict__ positions, int nh, int nkv, int hd, int page_size,
                int max_blocks, int num_pages, float scale, int window, int* status) {
    extern __shared__ float q_s[];  // [hd]
    __shared__ float p_s[CH];
    __shared__ int slot_s[CH];
    __shared__ float scratch[33];
    const int t = blockIdx.x, h = blockIdx.y, tid = threadIdx.x;
    const int kvh = h / (nh / nkv);
    const int seq = tok_seq[t];
    T* o = out + ((size_t)t * nh + h) * hd;
    if (seq < 0) {  // padding row of a fixed-shape batch
        for (int d = tid; d < hd; d += CH) o[d] = from_f<T>(0.f);
        return;
    }
    const int kv_end = positions[t] + 1;
    const int kv_begin = window > 0 ? max(0, kv_end - window) : 0;
    const T* qrow = q + (size_t)t * q_stride + (size_t)h * hd;
    for (int d = tid; d < hd; d += CH) q_s[d] = to_f(qrow[d]);
    __syncthreads();
    const int* table = block_tables + (size_t)seq * max_blocks;
    float m = -INFINITY, l = 0.f;
    float acc0 = 0.f, acc1 = 0.f;  // output dims tid and tid + CH (hd <= 256)
    for (int c0 = kv_begin; c0 < kv_end; c0 += CH) {
        const int j = c0 + tid;
        float s = -INFINITY;
        int slot = -1;
        if (j < kv_end) {
            const int blk = j / page_size;
            const int page = blk < max_blocks ? table[blk] : -1;
            if (page < 0 || page >= num_pages) {
                cw_report(status, CW_ST_PAGE_RANGE, t, page);
            } else {
                slot = page * page_size + j % page_size;
                const T* kp = k_cache + ((size_t)slot * nkv + kvh) * hd;
                float dot = 0.f;
                for (int d = 0; d < hd; ++d) dot = fmaf(q_s[d], to_f(kp[d]), dot);
                s = dot * scale;
            }
        }
        slot_s[tid] = slot;
        const float m_new = fmaxf(m, block_max(s, scratch));
        const float p = (slot >= 0) ? expf(s - m_new) : 0.f;
        p_s[tid] = p;
        const float csum = block_sum(p, scratch);  // also orders p_s/slot_s writes before reads
        const float alpha = (m == -INFINITY) ? 0.f : expf(m - m_new);
        l = l * alpha + csum;
        acc0 *= alpha;
        acc1 *= alpha;
        const int n = min(CH, kv_end - c0);
        if (m_new != -INFINITY) {
            for (int jj = 0; jj < n; ++jj) {
                const int sl = slot_s[jj];
                if (sl < 0) continue;
                const T* vp = v_cache + ((size_t)sl * nkv + kvh) * hd;
                const float pj = p_s[jj];
                if (tid < hd) acc0 = fmaf(pj, to_f(vp[tid]), acc0);
                if (tid + CH < hd) acc1 = fmaf(pj, to_f(vp[tid + CH]), acc1);
            }
            m = m_new;
        }
        __syncthreads();
    }
    const float inv = l > 0.f ? 1.0f / l : 0.f;
    if (tid < hd) o[tid] = from_f<T>(acc0 * inv);
    if (tid + CH < hd) o[tid + CH] = from_f<T>(acc1 * inv);
}

extern "C" int cw_attention_ref(const void* q, int q_stride, void* out, const void* k_cache,
                                const void* v_cache, const int* block_tables, const int* tok_seq,
                                const int* positions, int N, int nh, int nkv, int hd,
                                int page_size, int max_blocks, int num_pages, float scale,
                                int window, int dtype, int* status, cudaStream_t stream) {
    if (N == 0) return CW_OK;
    if (N < 0 || nh <= 0 || nkv <= 0 || nh % nkv != 0 || hd <= 0 || page_size <= 0 || max_blocks <= 0)
        return CW_ERR_BAD_SIZE;
    if (hd > 2 * CH || nh > 65535) return CW_ERR_UNSUPPORTED;
    dim3 grid(N, nh);
    const size_t smem = (size_t)hd * sizeof(float);
    if (dtype == 0)
        attn_ref_kernel<float><<<grid, CH, smem, stream>>>(
            (const float*)q, q_stride, (float*)out, (const float*)k_cache, (const float*)v_cache,
            block_tables, tok_seq, positions, nh, nkv, hd, page_size, max_blocks, num_pages, scale,
            window, status);
    else if (dtype == 1)
        attn_ref_kernel<bf16><<<grid, CH, smem, stream>>>(
            (const bf16*)q, q_stride, (bf16*)out, (const bf16*)k_cache, (const bf16*)v_cache,
            block_tables, tok_seq, positions, nh, nkv, hd, page_size, max_blocks, num_pages, scale,
            window, status);
    else
        return CW_ERR_BAD_DTYPE;
    return CW_LAUNCH_CHECK();
}

CW_TRACE_TU(attention_ref)
