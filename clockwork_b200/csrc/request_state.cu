// Per-request state on the device, and the kernel that turns it into a step's inputs.
//
// The reference keeps a request's progress and random generator on the host (Python fields of its
// Sequence and a CPU torch.Generator per request, clockwork/engine/model_runner.py:46, 139-145) and
// rebuilds every step's inputs there.  Here each running request owns a column of an int32 table on
// the device: {position, last token, draws, seed, temperature, top-k, top-p}.  A single-token step
// reads its inputs from that table: the token to feed is the one the last step sampled, the position
// is the request's progress, the cache slot follows from the position and the request's block table,
// and the uniform number of a stochastic draw is a pure function of (seed, draws).  The sampling
// kernels write the new token back and advance position and draws (sampling.cu: emit_token).  So a
// step can be launched before the host has read the step before it, and a step in which nothing but
// the positions changed needs no upload at all.
//
// The host can also overwrite a row's column at the start of a step (`fresh`): after a prompt, a
// preemption, or when the caller supplies the tokens itself (trace replay).
#include "common.cuh"

#define CW_RS_MAX_GROUPS 8

struct StepFromStateParams {
    const int* row_slot;  // [B] state slot of each row of the step; < 0: padding
    int* fresh;           // [B] 1: take the row's column from `fresh_values` first (cleared here)
    const int* fresh_values;  // [CW_RS_FIELDS][B]
    int* state;           // [CW_RS_FIELDS][num_slots]
    int num_slots, B, page_size, max_blocks, num_pages, num_groups;
    const int* tables[CW_RS_MAX_GROUPS];  // per page group: [B][max_blocks] block tables of the rows
    int* kv_slots[CW_RS_MAX_GROUPS];      // per page group: [B] cache slot of each row's token (out)
    int* tokens;      // [B] out
    int* positions;   // [B] out
    int* ctx_lens;    // [B] out: position + 1
    int* tok_seq;     // [B] out: the row itself, or -1 for padding
    float* temperature; int* top_k; float* top_p; float* uniform;  // [B] out
    int* status;
};

// The uniform number of draw `draw_index` of a request: 24 random bits from a splitmix64 mix of the
// seed and the counter.  clockwork_b200/sampling/sampler.py computes the same on the host.
__device__ __forceinline__ float uniform_for(unsigned long long seed, int draw_index) {
    unsigned long long z = seed * 0x9E3779B97F4A7C15ull + (unsigned long long)(draw_index + 1) * 0xD1B54A32D192ED03ull;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    z ^= z >> 31;
    return (float)(z >> 40) * (1.0f / 16777216.0f);
}

// The kernels of a step read its inputs (context lengths, block tables, ...) before they wait for their
// predecessors, taking them for settled when the step begins.  This kernel writes such inputs, so it
// must be complete before any other kernel of the step starts: it never releases its dependents early,
// and the kernel launched after it must be launched without the programmatic-serialization attribute
// (ops.embed(..., serial=True)), which makes the boundary behind this kernel an ordinary one.
__global__ void step_from_state_kernel(const StepFromStateParams p) {
    pdl_wait();  // the sampling kernel of the step before wrote the table
    const int r = blockIdx.x * blockDim.x + threadIdx.x;
    if (r >= p.B) return;
    const int slot = p.row_slot[r];
    if (slot < 0 || slot >= p.num_slots) {
        if (slot >= p.num_slots) cw_report(p.status, CW_ST_ROW_RANGE, r, slot);
        p.tokens[r] = 0;
        p.positions[r] = 0;
        p.ctx_lens[r] = 0;
        p.tok_seq[r] = -1;
        p.temperature[r] = 0.f;
        p.top_k[r] = 0;
        p.top_p[r] = 1.f;
        p.uniform[r] = 0.f;
        for (int g = 0; g < p.num_groups; ++g) p.kv_slots[g][r] = -1;
        return;
    }
    int* col = p.state + slot;
    if (p.fresh[r]) {
        for (int f = 0; f < CW_RS_FIELDS; ++f) col[f * p.num_slots] = p.fresh_values[f * p.B + r];
        p.fresh[r] = 0;
    }
    const int pos = col[CW_RS_POSITION * p.num_slots];
    p.tokens[r] = col[CW_RS_LAST_TOKEN * p.num_slots];
    p.positions[r] = pos;
    p.ctx_lens[r] = pos + 1;
    p.tok_seq[r] = r;
    p.temperature[r] = __int_as_float(col[CW_RS_TEMPERATURE * p.num_slots]);
    p.top_k[r] = col[CW_RS_TOP_K * p.num_slots];
    p.top_p[r] = __int_as_float(col[CW_RS_TOP_P * p.num_slots]);
    const unsigned long long seed = ((unsigned long long)(unsigned)col[CW_RS_SEED_HI * p.num_slots] << 32) |
                                    (unsigned)col[CW_RS_SEED_LO * p.num_slots];
    p.uniform[r] = uniform_for(seed, col[CW_RS_DRAWS * p.num_slots]);
    const int blk = pos / p.page_size, off = pos - blk * p.page_size;
    for (int g = 0; g < p.num_groups; ++g) {
        const int page = (pos >= 0 && blk < p.max_blocks) ? p.tables[g][(size_t)r * p.max_blocks + blk] : -1;
        if (page < 0 || page >= p.num_pages) {
            cw_report(p.status, CW_ST_PAGE_RANGE, r, page);
            p.kv_slots[g][r] = -1;
        } else {
            p.kv_slots[g][r] = page * p.page_size + off;
        }
    }
}

// tables / kv_slots: `num_groups` device pointers each (host arrays of pointers).
extern "C" int cw_step_from_state(const int* row_slot, int* fresh, const int* fresh_values, int* state, int num_slots,
                                  int B, int page_size, int max_blocks, int num_pages, int num_groups,
                                  const int* const* tables, int* const* kv_slots, int* tokens, int* positions,
                                  int* ctx_lens, int* tok_seq, float* temperature, int* top_k, float* top_p,
                                  float* uniform, int* status, cudaStream_t stream) {
    if (B == 0) return CW_OK;
    if (B < 0 || num_slots <= 0 || page_size <= 0 || max_blocks <= 0 || num_groups < 0 || num_groups > CW_RS_MAX_GROUPS)
        return CW_ERR_BAD_SIZE;
    StepFromStateParams p;
    p.row_slot = row_slot; p.fresh = fresh; p.fresh_values = fresh_values; p.state = state;
    p.num_slots = num_slots; p.B = B; p.page_size = page_size; p.max_blocks = max_blocks; p.num_pages = num_pages;
    p.num_groups = num_groups;
    for (int g = 0; g < CW_RS_MAX_GROUPS; ++g) {
        p.tables[g] = g < num_groups ? tables[g] : nullptr;
        p.kv_slots[g] = g < num_groups ? kv_slots[g] : nullptr;
    }
    p.tokens = tokens; p.positions = positions; p.ctx_lens = ctx_lens; p.tok_seq = tok_seq;
    p.temperature = temperature; p.top_k = top_k; p.top_p = top_p; p.uniform = uniform; p.status = status;
    const int threads = 64;
    return cw_launch(step_from_state_kernel, dim3((B + threads - 1) / threads), dim3(threads), 0, stream, 1, p);
}

CW_TRACE_TU(request_state)
