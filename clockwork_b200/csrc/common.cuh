// Shared helpers of the clockwork_b200 kernels (sm_100a only).
//
// Conventions of every exported entry point (all are extern "C", loaded with ctypes):
//   * pointers are device pointers owned by the caller; nothing here allocates;
//   * `dtype` is 0 for float32 and 1 for bfloat16 and names the type of activations,
//     matrices and caches; residual streams, logits, norm weights and biases are float32;
//   * `status` points to CW_STATUS_WORDS int32 words on the device; a kernel that meets an
//     index outside its table (token id, slot, page id) records the first such event there
//     and skips the access instead of faulting; the host checks it when it reads results;
//   * the last argument is the CUDA stream; the return value is a cudaError_t as int
//     (launch-configuration errors), or a negative CW_ERR_* code for refused sizes.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define CW_STATUS_WORDS 4
#define CW_OK 0
#define CW_ERR_BAD_SIZE (-1)
#define CW_ERR_BAD_DTYPE (-2)
#define CW_ERR_UNSUPPORTED (-3)

// status[0] codes
#define CW_ST_TOKEN_RANGE 1
#define CW_ST_SLOT_RANGE 2
#define CW_ST_PAGE_RANGE 3
#define CW_ST_WAIT_TIMEOUT 4
#define CW_ST_ROW_RANGE 5
#define CW_ST_SMEM_ALIGN 6
#define CW_ST_SPLIT_RANGE 7
#define CW_ST_SPLIT_BOUND 8

typedef __nv_bfloat16 bf16;

// Per-request state on the device (request_state.cu): an int32 table [CW_RS_FIELDS][num_slots], one
// column per request slot; the float fields are stored as their bits.
#define CW_RS_POSITION 0     // tokens of the request whose keys and values are in the cache = position of its next token
#define CW_RS_LAST_TOKEN 1   // the token to feed next (the one sampled last)
#define CW_RS_DRAWS 2        // tokens sampled so far: the counter of the request's random numbers
#define CW_RS_SEED_LO 3      // the request's 64-bit seed
#define CW_RS_SEED_HI 4
#define CW_RS_TEMPERATURE 5  // float; 0: greedy
#define CW_RS_TOP_K 6        // 0: off
#define CW_RS_TOP_P 7        // float
#define CW_RS_FIELDS 8

__device__ __forceinline__ void cw_report(int* status, int code, int a, int b) {
    if (status != nullptr && atomicCAS(&status[0], 0, code) == 0) {
        status[1] = a;
        status[2] = b;
    }
}

__device__ __forceinline__ float to_f(float x) { return x; }
__device__ __forceinline__ float to_f(bf16 x) { return __bfloat162float(x); }
template <typename T> __device__ __forceinline__ T from_f(float x);
template <> __device__ __forceinline__ float from_f<float>(float x) { return x; }
template <> __device__ __forceinline__ bf16 from_f<bf16>(float x) { return __float2bfloat16_rn(x); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Block-wide reductions with a fixed order (warp tree, then warp 0 over the warp results),
// so the result for a row never depends on what else is in the batch.
// `scratch` must hold 33 floats.  All threads receive the result.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nwarps = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    if (warp == 0) {
        float w = lane < nwarps ? scratch[lane] : 0.f;
        w = warp_sum(w);
        if (lane == 0) scratch[32] = w;
    }
    __syncthreads();
    return scratch[32];
}
__device__ __forceinline__ float block_max(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nwarps = (blockDim.x + 31) >> 5;
    v = warp_max(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    if (warp == 0) {
        float w = lane < nwarps ? scratch[lane] : -INFINITY;
        w = warp_max(w);
        if (lane == 0) scratch[32] = w;
    }
    __syncthreads();
    return scratch[32];
}

#define CW_LAUNCH_CHECK() ((int)cudaGetLastError())

// ---- programmatic dependent launch --------------------------------------------------------------
// Every kernel of the step is launched with the "programmatic stream serialization" attribute:
// it may be scheduled while its predecessor in the stream is still running.  The contract that
// keeps this correct: a kernel calls pdl_wait() before it reads anything a predecessor wrote and
// before it writes global memory at all; what it does before that (set-up, prefetching weights,
// which no kernel of the step writes) overlaps the predecessor's tail.  pdl_launch_dependents()
// at the top lets the successor do the same.  Both are no-ops in a kernel launched the plain way.
//
// Step timeline: when a trace buffer is set (cw_trace_set_* in every translation unit, normally null),
// thread 0 of every CTA notes the global timer at its start (in pdl_launch_dependents) and when a
// wait on the preceding kernel returns (in pdl_wait: the first time and the last time), and the
// kernels that call cw_trace_end() append one record when the CTA is done:
// {start, first release, last release, end, gridDim, blockIdx}.  The notes are kept in shared memory
// and the one atomic comes last, so that the timeline is not disturbed.  buf[0] counts records,
// buf[1] is the capacity, records of 8 words start at buf[8].
static __constant__ unsigned long long* cw_trace_ptr;
__device__ __forceinline__ unsigned long long* cw_trace_notes() {
    __shared__ unsigned long long notes[3];
    return notes;
}
__device__ __forceinline__ unsigned long long cw_globaltimer() {
    unsigned long long now;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
    return now;
}
__device__ __forceinline__ void cw_trace(unsigned phase) {
    if (cw_trace_ptr == nullptr || threadIdx.x != 0) return;
    unsigned long long* notes = cw_trace_notes();
    const unsigned long long now = cw_globaltimer();
    if (phase == 0) {
        notes[0] = now;
        notes[1] = notes[2] = 0;
    } else {
        if (notes[1] == 0) notes[1] = now;
        notes[2] = now;
    }
}
__device__ __forceinline__ void cw_trace_end() {
    unsigned long long* buf = cw_trace_ptr;
    if (buf == nullptr || threadIdx.x != 0) return;
    const unsigned long long* notes = cw_trace_notes();
    const unsigned long long now = cw_globaltimer();
    const unsigned long long i = atomicAdd(buf, 1ULL);
    if (i >= buf[1]) return;
    unsigned long long* rec = buf + 8 + 8 * i;
    rec[0] = notes[0];
    rec[1] = notes[1];
    rec[2] = notes[2];
    rec[3] = now;
    rec[4] = (unsigned long long)gridDim.x | ((unsigned long long)gridDim.y << 20) | ((unsigned long long)gridDim.z << 40);
    rec[5] = (unsigned long long)blockIdx.x | ((unsigned long long)blockIdx.y << 20) | ((unsigned long long)blockIdx.z << 40);
    unsigned smid;
    asm volatile("mov.u32 %0, %%smid;" : "=r"(smid));
    rec[6] = smid;
}
static inline int cw_trace_set_tu(void* buf) {
    return (int)cudaMemcpyToSymbol(cw_trace_ptr, &buf, sizeof(buf));
}
#define CW_TRACE_TU(name) \
    extern "C" int cw_trace_set_##name(void* buf) { return cw_trace_set_tu(buf); }

__device__ __forceinline__ void pdl_wait() {
    asm volatile("griddepcontrol.wait;" ::: "memory");
    cw_trace(1);
}
__device__ __forceinline__ void pdl_launch_dependents() {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    cw_trace(0);
}

// 1: launch with the attribute (default); 0: plain launches.  Set through cw_set_pdl().
extern "C" int cw_pdl_enabled();

template <typename... KArgs, typename... Args>
static inline int cw_launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                            unsigned cluster_z, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    int n = 0;
    if (cw_pdl_enabled()) {
        attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[n].val.programmaticStreamSerializationAllowed = 1;
        ++n;
    }
    if (cluster_z > 1) {
        attr[n].id = cudaLaunchAttributeClusterDimension;
        attr[n].val.clusterDim.x = 1;
        attr[n].val.clusterDim.y = 1;
        attr[n].val.clusterDim.z = cluster_z;
        ++n;
    }
    cfg.attrs = attr;
    cfg.numAttrs = n;
    const cudaError_t err = cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
    if (err != cudaSuccess) return (int)err;
    return (int)cudaGetLastError();
}
