// Greedy and stochastic sampling over float32 logits, one thread block per row.
//
// Reference: clockwork/engine/model_runner.py:134-164.  Greedy is the first maximal index
// (:136-137).  Otherwise logits are divided by the temperature (:149); top-k keeps logits not
// below the k-th largest (:150-152); top-p sorts descending, accumulates softmax mass and drops
// a token when the mass *before* it already exceeds top_p, so the token that crosses the
// threshold stays (:153-163); the token is then drawn from the softmax of what is left.
// The reference draws with torch.multinomial from a per-request generator; here the caller
// supplies one uniform number u in [0,1) per row and the token is the first index whose
// cumulative probability (in index order) exceeds u.
//
// Nothing is sorted: the k-th largest value and the top-p cut-off are found by a bitwise search
// over an order-preserving integer image of the logits (32 counting passes each).
#include "common.cuh"

#define ST 1024

__device__ __forceinline__ unsigned ordered_key(float f) {
    const unsigned b = __float_as_uint(f);
    return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}

// A sampled token leaves through here.  With a request-state table given (request_state.cu) the token
// also becomes the request's `last token`, and its position and draw counter advance by one: the next
// step can then be launched before the host has read this one's tokens.
__device__ __forceinline__ void emit_token(int row, int token, int* __restrict__ out, const int* __restrict__ row_slot,
                                           int* __restrict__ state, int num_slots) {
    out[row] = token;
    if (state != nullptr) {
        const int slot = row_slot[row];
        if (slot >= 0 && slot < num_slots) {
            state[CW_RS_LAST_TOKEN * num_slots + slot] = token;
            state[CW_RS_POSITION * num_slots + slot] += 1;
            state[CW_RS_DRAWS * num_slots + slot] += 1;
        }
    }
}

__global__ void __launch_bounds__(ST)
argmax_kernel(const float* __restrict__ logits, int* __restrict__ out, int V, size_t row_stride,
              const int* __restrict__ row_slot, int* __restrict__ state, int num_slots) {
    __shared__ float bv[32];
    __shared__ int bi[32];
    pdl_launch_dependents();
    pdl_wait();
    const float* row = logits + (size_t)blockIdx.x * row_stride;
    float best = -INFINITY;
    int idx = 0x7fffffff;
    for (int i = threadIdx.x; i < V; i += ST) {
        const float v = row[i];
        if (v > best || (v == best && i < idx)) { best = v; idx = i; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
        if (ov > best || (ov == best && oi < idx)) { best = ov; idx = oi; }
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (lane == 0) { bv[warp] = best; bi[warp] = idx; }
    __syncthreads();
    if (warp == 0) {
        best = bv[lane];
        idx = bi[lane];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best, o);
            const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
            if (ov > best || (ov == best && oi < idx)) { best = ov; idx = oi; }
        }
        if (lane == 0) emit_token(blockIdx.x, (idx == 0x7fffffff) ? 0 : idx, out, row_slot, state, num_slots);
    }
}

// row_slot / state (both or neither): see emit_token.
extern "C" int cw_argmax_state(const float* logits, int* out, int R, int V, long long row_stride, const int* row_slot,
                               int* state, int num_slots, cudaStream_t stream) {
    if (R == 0) return CW_OK;
    if (R < 0 || V <= 0 || row_stride < V || (state != nullptr && (row_slot == nullptr || num_slots <= 0))) return CW_ERR_BAD_SIZE;
    return cw_launch(argmax_kernel, dim3(R), dim3(ST), 0, stream, 1, logits, out, V, (size_t)row_stride, row_slot, state,
                     num_slots);
}

extern "C" int cw_argmax(const float* logits, int* out, int R, int V, long long row_stride,
                         cudaStream_t stream) {
    return cw_argmax_state(logits, out, R, V, row_stride, nullptr, nullptr, 0, stream);
}

__device__ __forceinline__ float block_sum_1024(float v, float* scratch) { return block_sum(v, scratch); }

__global__ void __launch_bounds__(ST)
sample_kernel(const float* __restrict__ logits, const float* __restrict__ temperature,
              const int* __restrict__ top_k, const float* __restrict__ top_p,
              const float* __restrict__ uniform, int* __restrict__ out, int V, size_t row_stride,
              const int* __restrict__ row_slot, int* __restrict__ state, int num_slots) {
    __shared__ float scratch[33];
    __shared__ float warp_tot[32];
    __shared__ int first_thread, last_thread;
    pdl_launch_dependents();
    pdl_wait();
    const int r = blockIdx.x, tid = threadIdx.x;
    const float* row = logits + (size_t)r * row_stride;
    const float temp = temperature[r];
    if (!(temp > 0.f)) {  // greedy row inside a mixed batch
        float best = -INFINITY;
        int idx = 0x7fffffff;
        for (int i = tid; i < V; i += ST) {
            const float v = row[i];
            if (v > best || (v == best && i < idx)) { best = v; idx = i; }
        }
        const float gmax = block_max(best, scratch);
        int cand = (best == gmax) ? idx : 0x7fffffff;
        if (tid == 0) first_thread = 0x7fffffff;
        __syncthreads();
        atomicMin(&first_thread, cand);
        __syncthreads();
        if (tid == 0) emit_token(r, first_thread == 0x7fffffff ? 0 : first_thread, out, row_slot, state, num_slots);
        return;
    }
    // pass 1: maximum of the scaled logits
    float mx = -INFINITY;
    for (int i = tid; i < V; i += ST) mx = fmaxf(mx, row[i] / temp);
    mx = block_max(mx, scratch);

    unsigned keep_key = 0u;  // a token is kept iff ordered_key(l) >= keep_key
    const int k = top_k[r];
    if (k > 0 && k < V) {
        unsigned thr = 0u;
        for (int bit = 31; bit >= 0; --bit) {
            const unsigned cand = thr | (1u << bit);
            float cnt = 0.f;
            for (int i = tid; i < V; i += ST) cnt += (ordered_key(row[i] / temp) >= cand) ? 1.f : 0.f;
            cnt = block_sum(cnt, scratch);
            if (cnt >= (float)k) thr = cand;
        }
        keep_key = thr;
    }
    const float p_lim = top_p[r];
    if (p_lim < 1.0f) {
        float zk = 0.f;
        for (int i = tid; i < V; i += ST) {
            const float l = row[i] / temp;
            if (ordered_key(l) >= keep_key) zk += expf(l - mx);
        }
        zk = block_sum(zk, scratch);
        // largest K0 whose strictly-greater mass still exceeds top_p; kept keys are > K0
        unsigned k0 = 0u;
        for (int bit = 31; bit >= 0; --bit) {
            const unsigned cand = k0 | (1u << bit);
            float g = 0.f;
            for (int i = tid; i < V; i += ST) {
                const float l = row[i] / temp;
                const unsigned key = ordered_key(l);
                if (key >= keep_key && key > cand) g += expf(l - mx);
            }
            g = block_sum(g, scratch);
            if (g > p_lim * zk) k0 = cand;
        }
        if (k0 != 0xffffffffu && k0 + 1u > keep_key) keep_key = k0 + 1u;
    }
    // final pass: inverse CDF in index order; thread t owns a contiguous range
    const int per = (V + ST - 1) / ST;
    const int lo = min(V, tid * per), hi = min(V, lo + per);
    float mine = 0.f;
    for (int i = lo; i < hi; ++i) {
        const float l = row[i] / temp;
        if (ordered_key(l) >= keep_key) mine += expf(l - mx);
    }
    // block-wide exclusive scan of `mine` in thread order
    const int lane = tid & 31, warp = tid >> 5;
    float incl = mine;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const float n = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += n;
    }
    if (lane == 31) warp_tot[warp] = incl;
    if (tid == 0) { first_thread = 0x7fffffff; last_thread = -1; }
    __syncthreads();
    float warp_off = 0.f, total = 0.f;
    for (int w = 0; w < 32; ++w) {
        if (w < warp) warp_off += warp_tot[w];
        total += warp_tot[w];
    }
    const float excl = warp_off + incl - mine;
    const float target = uniform[r] * total;
    if (mine > 0.f) {
        atomicMax(&last_thread, tid);
        if (excl + mine > target) atomicMin(&first_thread, tid);
    }
    __syncthreads();
    // when rounding leaves the target beyond the last kept token, the last owner takes it
    const int owner = first_thread != 0x7fffffff ? first_thread : last_thread;
    if (owner < 0) {
        if (tid == 0) emit_token(r, 0, out, row_slot, state, num_slots);
        return;
    }
    if (tid == owner) {
        float run = excl;
        int pick = -1, last_kept = lo;
        for (int i = lo; i < hi; ++i) {
            const float l = row[i] / temp;
            if (ordered_key(l) >= keep_key) {
                run += expf(l - mx);
                last_kept = i;
                if (run > target) { pick = i; break; }
            }
        }
        emit_token(r, pick >= 0 ? pick : last_kept, out, row_slot, state, num_slots);
    }
}

extern "C" int cw_sample_state(const float* logits, const float* temperature, const int* top_k, const float* top_p,
                               const float* uniform, int* out, int R, int V, long long row_stride, const int* row_slot,
                               int* state, int num_slots, cudaStream_t stream) {
    if (R == 0) return CW_OK;
    if (R < 0 || V <= 0 || row_stride < V || (state != nullptr && (row_slot == nullptr || num_slots <= 0))) return CW_ERR_BAD_SIZE;
    return cw_launch(sample_kernel, dim3(R), dim3(ST), 0, stream, 1, logits, temperature, top_k, top_p, uniform, out, V,
                     (size_t)row_stride, row_slot, state, num_slots);
}

extern "C" int cw_sample(const float* logits, const float* temperature, const int* top_k,
                         const float* top_p, const float* uniform, int* out, int R, int V,
                         long long row_stride, cudaStream_t stream) {
    return cw_sample_state(logits, temperature, top_k, top_p, uniform, out, R, V, row_stride, nullptr, nullptr, 0, stream);
}

CW_TRACE_TU(sampling)
