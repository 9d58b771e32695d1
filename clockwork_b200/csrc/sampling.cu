// Greedy and stochastic sampling over float32 logits, one thread block per row.
//
// Reference: clockwork/engine/model_runner.py:134-164.  Greedy is the first maximal index
// (:136-137).  Otherwise logits are divided by the temperature (:149); top-k keeps logits not
// below the k-th largest (:150-152); top-p sorts descending, accumulates softmax mass and drops
// a token when the mass *before* it already exceeds top_p, so the token that crosses the
// threshold stays (:153-163); the token is then drawn from the softmax of what is left.
// The reference draws with torch.multinomial from a per-request generator; here the caller
// supplies one uniform number u in [0,1) per row and the token is the first index whose
// cumulative probability (in index order) exceeds u.  Equal logits are kept or dropped together: under
// top-p a token stays iff the mass of the logits strictly above it does not exceed top_p (the reference's
// sort may cut between equal logits, in an order it does not define; every token it could keep stays here).
//
// Nothing is sorted: the k-th largest value and the top-p cut-off are found by a bitwise search
// over an order-preserving integer image of the logits (32 counting passes each).
#include "common.cuh"

#define ST 1024

__device__ __forceinline__ unsigned ordered_key(float f) {
    unsigned b = __float_as_uint(f);
    b = (b == 0x80000000u) ? 0u : b;  // -0.0 and +0.0 compare equal as floats: one image for both
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

// ---------------------------------------------------------------------------------------------
// The same rule over many thread blocks per row.
//
// sample_kernel above walks a row 65 times with one block: a vocabulary of 150,000 costs it a
// millisecond and more.  Here a row is cut into SP_BLOCKS chunks, a block each, and the two searches
// become radix selections over the order-preserving keys, 11 + 11 + 10 bits at a time, with
// histograms in global memory that every pass's blocks add to and the next pass's blocks read:
//   top-k: counts per bin; the bin in which the count from the top reaches k is refined;
//   top-p: mass per bin (of the keys top-k kept); the highest bin at which the mass from the top
//          exceeds top_p * Z is refined; the key found is the lowest one kept.
// Masses are integers, exp(l - max) * 2^40 truncated: sums of integers do not depend on the order in
// which blocks and threads add them up, so a row's token is the same on every run whatever the
// scheduling (floating-point atomics would not give that), and the final walk along the row in index
// order compares exact cumulative sums with u * total.  Workspace (zeroed before the first kernel):
// per row SP_WORDS 64-bit words.
// ---------------------------------------------------------------------------------------------
#define SP_THREADS 256
#define SP_BLOCKS 32
#define SP_L1 2048  // bins of key bits 31..21
#define SP_L2 2048  // bits 20..10
#define SP_L3 1024  // bits 9..0
#define SP_MASS_ONE 1099511627776.0f  // 2^40
// words of a row's workspace: [0] best (key << 32 | ~index), [1] Z, then counts (as 64-bit words, for one
// kind of atomic) and masses per level, then the blocks' kept mass
#define SP_CNT1 2
#define SP_CNT2 (SP_CNT1 + SP_L1)
#define SP_CNT3 (SP_CNT2 + SP_L2)
#define SP_MASS1 (SP_CNT3 + SP_L3)
#define SP_MASS2 (SP_MASS1 + SP_L1)
#define SP_MASS3 (SP_MASS2 + SP_L2)
#define SP_BLOCKSUM (SP_MASS3 + SP_L3)
#define SP_WORDS (SP_BLOCKSUM + SP_BLOCKS)

typedef unsigned long long u64;

__device__ __forceinline__ float key_to_float(unsigned key) {
    const unsigned b = (key & 0x80000000u) ? (key & 0x7fffffffu) : ~key;
    return __uint_as_float(b);
}
__device__ __forceinline__ u64 mass_of(float l, float mx) { return (u64)(expf(l - mx) * SP_MASS_ONE); }

struct SampleParams {
    const float* logits; size_t row_stride; int V;
    const float* temperature; const int* top_k; const float* top_p; const float* uniform;
    u64* work;  // [rows][SP_WORDS]
    int* out; const int* row_slot; int* state; int num_slots;
};

// Walks a histogram of `bins` 64-bit words from the top and finds the bin at which the running sum
// first satisfies the rule: counts, sum >= want (the want-th largest key lies in it); masses, sum >
// want.  Returns the bin (the lowest one if rounding lets none qualify) and leaves the sum above it in
// *above.  Every thread of the block calls it and gets the same answer.  `scratch`: 16 words.
__device__ int find_bin(const u64* hist, int bins, double want, bool strictly, u64* above, u64* scratch) {
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, per = bins / SP_THREADS;
    // thread 0 owns the highest bins; an inclusive scan over the threads' sums, from the top down
    u64 mine = 0;
    for (int j = 0; j < per; ++j) mine += hist[bins - 1 - (tid * per + j)];
    u64 incl = mine;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const u64 n = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += n;
    }
    if (lane == 31) scratch[warp] = incl;
    if (tid == 0) scratch[8] = (u64)0xffffffffu;  // the first thread whose sum qualifies
    __syncthreads();
    u64 before = 0;
    for (int w = 0; w < warp; ++w) before += scratch[w];
    incl += before;
    const bool ok = strictly ? (double)incl > want : (double)incl >= want;
    if (ok) atomicMin((unsigned*)&scratch[8], (unsigned)tid);
    __syncthreads();
    const int owner = (int)(unsigned)scratch[8];
    if (tid == (owner < SP_THREADS ? owner : SP_THREADS - 1)) {
        u64 run = incl - mine;
        int bin = 0;
        bool found = false;
        for (int j = 0; j < per && !found; ++j) {
            const int c = bins - 1 - (tid * per + j);
            const u64 next = run + hist[c];
            if (strictly ? (double)next > want : (double)next >= want) {
                bin = c;
                found = true;
            } else {
                run = next;
            }
        }
        if (!found) {  // (rounding: take the lowest bin, with everything above it)
            bin = 0;
            run = incl - hist[0];
        }
        scratch[9] = (u64)bin;
        scratch[10] = run;
    }
    __syncthreads();
    const int bin = (int)scratch[9];
    *above = scratch[10];
    __syncthreads();
    return bin;
}

// What a pass settles (the bits of the key found so far, and what is still wanted inside them) is kept
// in the row's workspace, a pair of words per pass: pass n reads what pass n - 1 left and leaves its own
// (every block computes the same; block 0 writes it).
#define SP_STATE (SP_BLOCKSUM + SP_BLOCKS)
#undef SP_WORDS
#define SP_WORDS (SP_STATE + 16)

// PASS 0: best (largest key, first index) of every row, and top-k's counts of key bits 31..21.
//      1, 2: top-k's counts of the next bits, inside the bins found so far.
//      3: top-k settled (its lowest key kept: state word 6); top-p's masses of bits 31..21 and Z.
//      4, 5: top-p's masses of the next bits.
//      6: top-p settled (the lowest key kept at all: state word 12); the blocks' kept mass.
template <int PASS>
__global__ void __launch_bounds__(SP_THREADS)
sample_pass_kernel(const SampleParams p) {
    __shared__ u64 hist[SP_L1];
    __shared__ u64 scratch[16];
    pdl_launch_dependents();
    pdl_wait();
    const int r = blockIdx.y, tid = threadIdx.x;
    const float temp = p.temperature[r];
    const bool sampled = temp > 0.f;
    if (PASS > 0 && !sampled) return;  // (a greedy row needs its best only)
    const float* row = p.logits + (size_t)r * p.row_stride;
    u64* w = p.work + (size_t)r * SP_WORDS;
    u64* state = w + SP_STATE;
    const int chunk = (p.V + SP_BLOCKS - 1) / SP_BLOCKS;
    const int lo = min(p.V, (int)blockIdx.x * chunk), hi = min(p.V, lo + chunk);
    const int k = p.top_k[r];
    const bool by_k = sampled && k > 0 && k < p.V;
    const float lim = p.top_p[r];
    const bool by_p = sampled && lim < 1.0f;

    // ---- what the passes before this one settled --------------------------------------------------
    unsigned prefix = 0u, keep_k = 0u, keep = 0u;
    if (PASS == 1 || PASS == 2 || PASS == 3) {
        if (by_k) {
            double want = PASS == 1 ? (double)k : __longlong_as_double((long long)state[2 * (PASS - 1) + 1]);
            prefix = PASS == 1 ? 0u : (unsigned)state[2 * (PASS - 1)];
            u64 above;
            const int bin = find_bin(w + (PASS == 1 ? SP_CNT1 : (PASS == 2 ? SP_CNT2 : SP_CNT3)), PASS == 3 ? SP_L3 : SP_L1, want,
                                     false, &above, scratch);
            want -= (double)above;
            prefix |= (unsigned)bin << (PASS == 1 ? 21 : (PASS == 2 ? 10 : 0));
            if (PASS == 3) keep_k = prefix;
            if (blockIdx.x == 0 && tid == 0) {
                state[2 * PASS] = prefix;
                state[2 * PASS + 1] = (u64)__double_as_longlong(want);
            }
        } else if (PASS == 3 && blockIdx.x == 0 && tid == 0) {
            state[6] = 0u;
        }
        if (PASS < 3 && !by_k) return;
    }
    if (PASS >= 4) {
        keep_k = (unsigned)state[6];
        if (by_p) {
            double want = PASS == 4 ? (double)lim * (double)w[1] : __longlong_as_double((long long)state[2 * (PASS - 1) + 1]);
            prefix = PASS == 4 ? 0u : (unsigned)state[2 * (PASS - 1)];
            u64 above;
            const int bin = find_bin(w + (PASS == 4 ? SP_MASS1 : (PASS == 5 ? SP_MASS2 : SP_MASS3)), PASS == 6 ? SP_L3 : SP_L1, want,
                                     true, &above, scratch);
            want -= (double)above;
            prefix |= (unsigned)bin << (PASS == 4 ? 21 : (PASS == 5 ? 10 : 0));
            if (blockIdx.x == 0 && tid == 0) {
                state[2 * PASS] = prefix;
                state[2 * PASS + 1] = (u64)__double_as_longlong(want);
            }
        } else if (PASS < 6) {
            return;
        }
        if (PASS == 6) keep = by_p ? max(keep_k, prefix) : keep_k;
    }
    if (PASS == 3 && !by_p) return;

    // ---- this pass's walk over the block's part of the row ------------------------------------------
    if (PASS != 6)
        for (int i = tid; i < SP_L1; i += SP_THREADS) hist[i] = 0;
    __syncthreads();
    const float mx = PASS >= 3 ? key_to_float((unsigned)(w[0] >> 32)) : 0.f;
    u64 best = 0, total = 0;
    for (int i = lo + tid; i < hi; i += SP_THREADS) {
        const float l = sampled ? row[i] / temp : row[i];
        const unsigned key = ordered_key(l);
        if (PASS == 0) {
            const u64 cand = ((u64)key << 32) | (u64)(~(unsigned)i);
            best = cand > best ? cand : best;
            if (by_k) atomicAdd(&hist[key >> 21], 1ULL);
        } else if (PASS == 1) {
            if ((key >> 21) == (prefix >> 21)) atomicAdd(&hist[(key >> 10) & (SP_L2 - 1)], 1ULL);
        } else if (PASS == 2) {
            if ((key >> 10) == (prefix >> 10)) atomicAdd(&hist[key & (SP_L3 - 1)], 1ULL);
        } else if (PASS == 3) {
            if (key >= keep_k) {
                const u64 q = mass_of(l, mx);
                total += q;
                atomicAdd(&hist[key >> 21], q);
            }
        } else if (PASS == 4) {
            if (key >= keep_k && (key >> 21) == (prefix >> 21)) atomicAdd(&hist[(key >> 10) & (SP_L2 - 1)], mass_of(l, mx));
        } else if (PASS == 5) {
            if (key >= keep_k && (key >> 10) == (prefix >> 10)) atomicAdd(&hist[key & (SP_L3 - 1)], mass_of(l, mx));
        } else {
            if (key >= keep) total += mass_of(l, mx);
        }
    }
    __syncthreads();
    // ---- the block's share goes to the row's workspace -------------------------------------------------
    if (PASS == 0) {
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const u64 other = __shfl_xor_sync(0xffffffffu, best, o);
            best = other > best ? other : best;
        }
        if ((tid & 31) == 0 && best != 0) atomicMax(&w[0], best);
    }
    if (PASS == 3 || PASS == 6) {
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) total += __shfl_xor_sync(0xffffffffu, total, o);
        if ((tid & 31) == 0) scratch[tid >> 5] = total;
        __syncthreads();
        if (tid == 0) {
            u64 t = 0;
            for (int i = 0; i < SP_THREADS / 32; ++i) t += scratch[i];
            if (PASS == 3) {
                atomicAdd(&w[1], t);
            } else {
                w[SP_BLOCKSUM + blockIdx.x] = t;
                if (blockIdx.x == 0) state[12] = keep;
            }
        }
    }
    if (PASS != 6 && (PASS != 0 || by_k)) {
        constexpr int OUT = PASS == 0 ? SP_CNT1 : (PASS == 1 ? SP_CNT2 : (PASS == 2 ? SP_CNT3 : (PASS == 3 ? SP_MASS1 : (PASS == 4 ? SP_MASS2 : SP_MASS3))));
        constexpr int NB = (PASS == 2 || PASS == 5) ? SP_L3 : SP_L1;
        for (int i = tid; i < NB; i += SP_THREADS)
            if (hist[i] != 0) atomicAdd(&w[OUT + i], hist[i]);
    }
}

// The last kernel of the chain, a block per row: the token.  A greedy row's is its best; a sampled row's
// is the first index, in index order, at which the kept mass so far exceeds u * total: the block of the
// row in which that happens follows from the blocks' sums, and that block's part of the row is walked.
__global__ void __launch_bounds__(SP_THREADS)
sample_pick_kernel(const SampleParams p) {
    __shared__ u64 warp_tot[SP_THREADS / 32];
    __shared__ int first_thread;
    pdl_launch_dependents();
    pdl_wait();
    const int r = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const u64* w = p.work + (size_t)r * SP_WORDS;
    const int best_index = (int)(~(unsigned)(w[0] & 0xffffffffu));
    const float temp = p.temperature[r];
    if (!(temp > 0.f) || w[0] == 0) {
        if (tid == 0) emit_token(r, w[0] == 0 ? 0 : best_index, p.out, p.row_slot, p.state, p.num_slots);
        return;
    }
    const unsigned keep = (unsigned)w[SP_STATE + 12];
    const float mx = key_to_float((unsigned)(w[0] >> 32));
    u64 total = 0;
    for (int b = 0; b < SP_BLOCKS; ++b) total += w[SP_BLOCKSUM + b];
    const double target = (double)p.uniform[r] * (double)total;
    int part = -1;
    u64 base = 0;
    for (int b = 0; b < SP_BLOCKS && part < 0; ++b) {
        const u64 next = base + w[SP_BLOCKSUM + b];
        if ((double)next > target)
            part = b;
        else
            base = next;
    }
    if (part < 0) {  // (no mass at all: cannot happen while the best key's mass is 2^40)
        if (tid == 0) emit_token(r, best_index, p.out, p.row_slot, p.state, p.num_slots);
        return;
    }
    const float* row = p.logits + (size_t)r * p.row_stride;
    const int chunk = (p.V + SP_BLOCKS - 1) / SP_BLOCKS;
    const int lo = min(p.V, part * chunk), hi = min(p.V, lo + chunk);
    const int per = (hi - lo + SP_THREADS - 1) / SP_THREADS;
    const int my_lo = min(hi, lo + tid * per), my_hi = min(hi, my_lo + per);
    u64 mine = 0;
    for (int i = my_lo; i < my_hi; ++i) {
        const float l = row[i] / temp;
        if (ordered_key(l) >= keep) mine += mass_of(l, mx);
    }
    u64 incl = mine;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const u64 n = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += n;
    }
    if (lane == 31) warp_tot[warp] = incl;
    if (tid == 0) first_thread = SP_THREADS;
    __syncthreads();
    u64 before = base;
    for (int wi = 0; wi < warp; ++wi) before += warp_tot[wi];
    incl += before;
    if (mine > 0 && (double)incl > target) atomicMin(&first_thread, tid);
    __syncthreads();
    if (tid == first_thread) {
        u64 run = incl - mine;
        int pick = my_lo;
        for (int i = my_lo; i < my_hi; ++i) {
            const float l = row[i] / temp;
            if (ordered_key(l) >= keep) {
                run += mass_of(l, mx);
                pick = i;
                if ((double)run > target) break;
            }
        }
        emit_token(r, pick, p.out, p.row_slot, p.state, p.num_slots);
    } else if (first_thread == SP_THREADS && tid == 0) {
        emit_token(r, best_index, p.out, p.row_slot, p.state, p.num_slots);  // (unreachable: the part's sum exceeds the target)
    }
}

// Words of workspace that cw_sample_rows needs for R rows (64-bit words).
extern "C" long long cw_sample_workspace_words(int R) { return (long long)(R > 0 ? R : 0) * SP_WORDS; }

// As cw_sample_state, over SP_BLOCKS thread blocks per row: `work` holds cw_sample_workspace_words(R)
// 64-bit words, which this call zeroes first.
extern "C" int cw_sample_rows(const float* logits, const float* temperature, const int* top_k, const float* top_p,
                              const float* uniform, int* out, int R, int V, long long row_stride, const int* row_slot,
                              int* state, int num_slots, unsigned long long* work, cudaStream_t stream) {
    if (R == 0) return CW_OK;
    if (R < 0 || V <= 0 || row_stride < V || work == nullptr || (state != nullptr && (row_slot == nullptr || num_slots <= 0)))
        return CW_ERR_BAD_SIZE;
    if (R > 65535) return CW_ERR_BAD_SIZE;
    if (cudaMemsetAsync(work, 0, (size_t)R * SP_WORDS * sizeof(u64), stream) != cudaSuccess) return (int)cudaGetLastError();
    SampleParams p;
    p.logits = logits; p.row_stride = (size_t)row_stride; p.V = V;
    p.temperature = temperature; p.top_k = top_k; p.top_p = top_p; p.uniform = uniform;
    p.work = work; p.out = out; p.row_slot = row_slot; p.state = state; p.num_slots = num_slots;
    const dim3 grid(SP_BLOCKS, R), block(SP_THREADS);
    int rc;
#define CW_PASS(n) \
    if ((rc = cw_launch(sample_pass_kernel<n>, grid, block, 0, stream, 1, p)) != CW_OK) return rc;
    CW_PASS(0) CW_PASS(1) CW_PASS(2) CW_PASS(3) CW_PASS(4) CW_PASS(5) CW_PASS(6)
#undef CW_PASS
    return cw_launch(sample_pick_kernel, dim3(R), block, 0, stream, 1, p);
}

CW_TRACE_TU(sampling)
