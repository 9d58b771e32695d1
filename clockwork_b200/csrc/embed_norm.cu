// Embedding gather and fused residual-add + RMSNorm.
//
// Reference formulas: clockwork/engine/model.py:200 (embedding), :44-49 (RMSNorm: float32
// statistics, x * rsqrt(mean(x^2) + eps), then the weight), :150 and :154 (residual sums).
// The residual stream is float32 in both run precisions; the normed output has the run's
// activation type.
#include "common.cuh"

template <typename T>
__global__ void embed_kernel(float* __restrict__ out, const T* __restrict__ table,
                             const int* __restrict__ ids, int H, int V, int* status) {
    pdl_launch_dependents();
    pdl_wait();
    const int row = blockIdx.x;
    const int id = ids[row];
    float* o = out + (size_t)row * H;
    if (id < 0 || id >= V) {
        if (threadIdx.x == 0) cw_report(status, CW_ST_TOKEN_RANGE, row, id);
        for (int c = threadIdx.x; c < H; c += blockDim.x) o[c] = 0.f;
        return;
    }
    const T* src = table + (size_t)id * H;
    for (int c = threadIdx.x; c < H; c += blockDim.x) o[c] = to_f(src[c]);
}

extern "C" int cw_embed(float* out, const void* table, const int* ids, int N, int H, int V,
                        int dtype, int* status, cudaStream_t stream) {
    if (N == 0) return CW_OK;
    if (N < 0 || H <= 0 || V <= 0) return CW_ERR_BAD_SIZE;
    const int threads = H >= 1024 ? 256 : 128;
    if (dtype == 0)
        return cw_launch(embed_kernel<float>, dim3(N), dim3(threads), 0, stream, 1, out, (const float*)table, ids, H, V, status);
    if (dtype == 1)
        return cw_launch(embed_kernel<bf16>, dim3(N), dim3(threads), 0, stream, 1, out, (const bf16*)table, ids, H, V, status);
    return CW_ERR_BAD_DTYPE;
}

// resid[row] (+= delta[row]); out[r] = weight * (x * rsqrt(mean(x^2)+eps)).
// With `rows` given, output row r is computed from residual row rows[r] (no add is done).
template <typename T>
__global__ void add_rmsnorm_kernel(float* __restrict__ resid, const T* __restrict__ delta,
                                   const float* __restrict__ weight, T* __restrict__ out,
                                   const int* __restrict__ rows, int num_resid_rows, float eps,
                                   int H, int* status) {
    __shared__ float scratch[33];
    pdl_launch_dependents();
    pdl_wait();
    const int r = blockIdx.x;
    int src_row = r;
    if (rows != nullptr) {
        src_row = rows[r];
        if (src_row < 0 || src_row >= num_resid_rows) {
            if (threadIdx.x == 0) cw_report(status, CW_ST_ROW_RANGE, r, src_row);
            for (int c = threadIdx.x; c < H; c += blockDim.x) out[(size_t)r * H + c] = from_f<T>(0.f);
            return;
        }
    }
    float* x = resid + (size_t)src_row * H;
    const T* d = delta ? delta + (size_t)src_row * H : nullptr;
    float ss = 0.f;
    for (int c = threadIdx.x; c < H; c += blockDim.x) {
        float v = x[c];
        if (d) {
            v += to_f(d[c]);
            x[c] = v;
        }
        ss = fmaf(v, v, ss);
    }
    ss = block_sum(ss, scratch);
    const float inv = 1.0f / sqrtf(ss / (float)H + eps);
    T* o = out + (size_t)r * H;
    for (int c = threadIdx.x; c < H; c += blockDim.x) o[c] = from_f<T>(weight[c] * (x[c] * inv));
}

// The same for many rows (prompt portions): one warp per row, the row held in registers between the
// sum of squares and the scaling, 16-byte accesses, no block-level synchronisation.  H must be a
// multiple of 4 and at most 128 * NV.
template <typename T>
struct Vec4;
template <>
struct Vec4<float> {
    static __device__ __forceinline__ float4 load(const float* p) { return *reinterpret_cast<const float4*>(p); }
    static __device__ __forceinline__ void store(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
};
template <>
struct Vec4<bf16> {
    static __device__ __forceinline__ float4 load(const bf16* p) {
        const uint2 r = *reinterpret_cast<const uint2*>(p);
        const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&r.x), b = *reinterpret_cast<const __nv_bfloat162*>(&r.y);
        return make_float4(__low2float(a), __high2float(a), __low2float(b), __high2float(b));
    }
    static __device__ __forceinline__ void store(bf16* p, float4 v) {
        const __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
        uint2 r;
        r.x = *reinterpret_cast<const uint32_t*>(&a);
        r.y = *reinterpret_cast<const uint32_t*>(&b);
        *reinterpret_cast<uint2*>(p) = r;
    }
};

template <typename T, int NV>
__global__ void __launch_bounds__(256)
add_rmsnorm_warp_kernel(float* __restrict__ resid, const T* __restrict__ delta, const float* __restrict__ weight,
                        T* __restrict__ out, int num_rows, float eps, int H) {
    pdl_launch_dependents();
    pdl_wait();
    const int lane = threadIdx.x & 31;
    const int r = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (r >= num_rows) return;
    float* x = resid + (size_t)r * H;
    const T* d = delta ? delta + (size_t)r * H : nullptr;
    float4 v[NV];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        const int c = (i * 32 + lane) * 4;
        if (c < H) {
            v[i] = Vec4<float>::load(x + c);
            if (d) {
                const float4 dv = Vec4<T>::load(d + c);
                v[i].x += dv.x; v[i].y += dv.y; v[i].z += dv.z; v[i].w += dv.w;
                Vec4<float>::store(x + c, v[i]);
            }
            ss = fmaf(v[i].x, v[i].x, ss); ss = fmaf(v[i].y, v[i].y, ss);
            ss = fmaf(v[i].z, v[i].z, ss); ss = fmaf(v[i].w, v[i].w, ss);
        }
    }
    ss = warp_sum(ss);
    const float inv = 1.0f / sqrtf(ss / (float)H + eps);
    T* o = out + (size_t)r * H;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        const int c = (i * 32 + lane) * 4;
        if (c < H) {
            const float4 w = Vec4<float>::load(weight + c);
            Vec4<T>::store(o + c, make_float4(w.x * (v[i].x * inv), w.y * (v[i].y * inv), w.z * (v[i].z * inv), w.w * (v[i].w * inv)));
        }
    }
}

template <typename T>
static int launch_rmsnorm_warp(float* resid, const T* delta, const float* weight, T* out, int rows, int H, float eps,
                               cudaStream_t stream) {
    const int warps = 8;
    const dim3 grid((rows + warps - 1) / warps), block(warps * 32);
    const int nv = (H + 127) / 128;
#define CW_NV(n) \
    if (nv <= n) return cw_launch(add_rmsnorm_warp_kernel<T, n>, grid, block, 0, stream, 1, resid, delta, weight, out, rows, eps, H);
    CW_NV(4) CW_NV(8) CW_NV(12) CW_NV(16) CW_NV(24) CW_NV(32)
#undef CW_NV
    return CW_ERR_UNSUPPORTED;
}

extern "C" int cw_add_rmsnorm(float* resid, const void* delta, const float* weight, void* out,
                              const int* rows, int num_out_rows, int num_resid_rows, int H,
                              float eps, int dtype, int* status, cudaStream_t stream) {
    if (num_out_rows == 0) return CW_OK;
    if (num_out_rows < 0 || H <= 0) return CW_ERR_BAD_SIZE;
    if (rows != nullptr && delta != nullptr) return CW_ERR_UNSUPPORTED;
    // many rows: a warp per row; few rows (decode): a block per row, for the latency of the one row
    const bool aligned = H % 4 == 0 && H <= 4096 && ((uintptr_t)resid & 15) == 0 && ((uintptr_t)weight & 15) == 0 &&
                         ((uintptr_t)out & 15) == 0 && ((uintptr_t)delta & 15) == 0;
    if (rows == nullptr && num_out_rows >= 256 && aligned) {
        if (dtype == 0)
            return launch_rmsnorm_warp<float>(resid, (const float*)delta, weight, (float*)out, num_out_rows, H, eps, stream);
        if (dtype == 1)
            return launch_rmsnorm_warp<bf16>(resid, (const bf16*)delta, weight, (bf16*)out, num_out_rows, H, eps, stream);
        return CW_ERR_BAD_DTYPE;
    }
    const int threads = H >= 2048 ? 512 : (H >= 512 ? 256 : 128);
    if (dtype == 0)
        return cw_launch(add_rmsnorm_kernel<float>, dim3(num_out_rows), dim3(threads), 0, stream, 1, resid,
                         (const float*)delta, weight, (float*)out, rows, num_resid_rows, eps, H, status);
    if (dtype == 1)
        return cw_launch(add_rmsnorm_kernel<bf16>, dim3(num_out_rows), dim3(threads), 0, stream, 1, resid,
                         (const bf16*)delta, weight, (bf16*)out, rows, num_resid_rows, eps, H, status);
    return CW_ERR_BAD_DTYPE;
}

// resid[r] += parts[0][r] + parts[1][r] + .. (in this order: the splits of a product over K that were
// kept apart), then, with `out`, out[r] = resid[r] normalised as above.  A warp per row, the row in
// registers between the two passes.
template <typename T, int NV>
__global__ void __launch_bounds__(256)
add_parts_rmsnorm_kernel(float* __restrict__ resid, const float* __restrict__ parts, int num_parts, size_t part_stride,
                         const float* __restrict__ weight, T* __restrict__ out, int num_rows, float eps, int H) {
    pdl_launch_dependents();
    pdl_wait();
    const int lane = threadIdx.x & 31;
    const int r = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (r >= num_rows) return;
    float* x = resid + (size_t)r * H;
    float4 v[NV];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        const int c = (i * 32 + lane) * 4;
        if (c < H) v[i] = Vec4<float>::load(x + c);
    }
    for (int k = 0; k < num_parts; ++k) {
        const float* d = parts + k * part_stride + (size_t)r * H;
#pragma unroll
        for (int i = 0; i < NV; ++i) {
            const int c = (i * 32 + lane) * 4;
            if (c < H) {
                const float4 dv = Vec4<float>::load(d + c);
                v[i].x += dv.x; v[i].y += dv.y; v[i].z += dv.z; v[i].w += dv.w;
            }
        }
    }
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        const int c = (i * 32 + lane) * 4;
        if (c < H) {
            Vec4<float>::store(x + c, v[i]);
            ss = fmaf(v[i].x, v[i].x, ss); ss = fmaf(v[i].y, v[i].y, ss);
            ss = fmaf(v[i].z, v[i].z, ss); ss = fmaf(v[i].w, v[i].w, ss);
        }
    }
    if (out == nullptr) return;
    ss = warp_sum(ss);
    const float inv = 1.0f / sqrtf(ss / (float)H + eps);
    T* o = out + (size_t)r * H;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        const int c = (i * 32 + lane) * 4;
        if (c < H) {
            const float4 w = Vec4<float>::load(weight + c);
            Vec4<T>::store(o + c, make_float4(w.x * (v[i].x * inv), w.y * (v[i].y * inv), w.z * (v[i].z * inv), w.w * (v[i].w * inv)));
        }
    }
}

template <typename T>
static int launch_add_parts(float* resid, const float* parts, int num_parts, size_t part_stride, const float* weight, T* out,
                            int rows, int H, float eps, cudaStream_t stream) {
    const int warps = 8;
    const dim3 grid((rows + warps - 1) / warps), block(warps * 32);
    const int nv = (H + 127) / 128;
#define CW_NV(n) \
    if (nv <= n) return cw_launch(add_parts_rmsnorm_kernel<T, n>, grid, block, 0, stream, 1, resid, parts, num_parts, part_stride, weight, out, rows, eps, H);
    CW_NV(4) CW_NV(8) CW_NV(12) CW_NV(16) CW_NV(24) CW_NV(32)
#undef CW_NV
    return CW_ERR_UNSUPPORTED;
}

// parts: float32 [num_parts][part_rows][H] (part_rows >= rows); out null: only the sum.  H a multiple of 4,
// at most 4096; 16-byte aligned pointers; CW_ERR_UNSUPPORTED otherwise.
extern "C" int cw_add_parts_rmsnorm(float* resid, const float* parts, int num_parts, int part_rows, const float* weight,
                                    void* out, int rows, int H, float eps, int dtype, cudaStream_t stream) {
    if (rows == 0) return CW_OK;
    if (rows < 0 || H <= 0 || num_parts < 1 || part_rows < rows) return CW_ERR_BAD_SIZE;
    if (H % 4 != 0 || H > 4096 || ((uintptr_t)resid & 15) || ((uintptr_t)parts & 15) || ((uintptr_t)weight & 15) ||
        ((uintptr_t)out & 15))
        return CW_ERR_UNSUPPORTED;
    const size_t stride = (size_t)part_rows * H;
    if (out == nullptr || dtype == 0)
        return launch_add_parts<float>(resid, parts, num_parts, stride, weight, (float*)out, rows, H, eps, stream);
    if (dtype == 1) return launch_add_parts<bf16>(resid, parts, num_parts, stride, weight, (bf16*)out, rows, H, eps, stream);
    return CW_ERR_BAD_DTYPE;
}

// out = silu(gate) * up, gate and up being the two halves of each row of `gate_up` [N, 2*I]
// (clockwork/engine/model.py:62-63).  Used where the product is not fused into the GEMM.
template <typename T>
__global__ void silu_mul_kernel(const T* __restrict__ gate_up, T* __restrict__ out, int I,
                                size_t total) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const size_t row = i / I, col = i % I;
    const float g = to_f(gate_up[row * 2 * I + col]);
    const float u = to_f(gate_up[row * 2 * I + I + col]);
    out[i] = from_f<T>(g / (1.0f + expf(-g)) * u);
}

extern "C" int cw_silu_mul(const void* gate_up, void* out, int N, int I, int dtype,
                           cudaStream_t stream) {
    if (N == 0) return CW_OK;
    if (N < 0 || I <= 0) return CW_ERR_BAD_SIZE;
    const size_t total = (size_t)N * I;
    const int threads = 256;
    const unsigned blocks = (unsigned)((total + threads - 1) / threads);
    if (dtype == 0)
        silu_mul_kernel<float><<<blocks, threads, 0, stream>>>((const float*)gate_up, (float*)out, I, total);
    else if (dtype == 1)
        silu_mul_kernel<bf16><<<blocks, threads, 0, stream>>>((const bf16*)gate_up, (bf16*)out, I, total);
    else
        return CW_ERR_BAD_DTYPE;
    return CW_LAUNCH_CHECK();
}

// resid += delta (float32 += T); used where a part returns a delta that no norm follows.
template <typename T>
__global__ void add_to_residual_kernel(float* __restrict__ resid, const T* __restrict__ delta,
                                       size_t total) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < total) resid[i] += to_f(delta[i]);
}

extern "C" int cw_add_to_residual(float* resid, const void* delta, int N, int H, int dtype,
                                  cudaStream_t stream) {
    if (N == 0) return CW_OK;
    if (N < 0 || H <= 0) return CW_ERR_BAD_SIZE;
    const size_t total = (size_t)N * H;
    const unsigned blocks = (unsigned)((total + 255) / 256);
    if (dtype == 0)
        add_to_residual_kernel<float><<<blocks, 256, 0, stream>>>(resid, (const float*)delta, total);
    else if (dtype == 1)
        add_to_residual_kernel<bf16><<<blocks, 256, 0, stream>>>(resid, (const bf16*)delta, total);
    else
        return CW_ERR_BAD_DTYPE;
    return CW_LAUNCH_CHECK();
}

static int g_pdl = 1;
extern "C" int cw_pdl_enabled() { return g_pdl; }
extern "C" int cw_set_pdl(int on) { g_pdl = on ? 1 : 0; return CW_OK; }

CW_TRACE_TU(embed_norm)
