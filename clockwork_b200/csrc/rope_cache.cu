// Rotary position encoding fused with the slot-mapped write of K and V into the paged cache,
// and the page copy that copy-on-write needs.
//
// Reference: clockwork/engine/model.py:92-95 (q*cos + rotate_half(q)*sin, element j paired
// with j + rotary_dim/2, cos/sin broadcast over heads), :186-191 (angle = float(position) *
// inv_freq[j], in float32), clockwork/kvcache/kv_cache.py:37-45 (scatter by slot, slot =
// page*page_size + position % page_size) and :32-35 (copy of one page in every layer).
// The rotation is done in float32 from float32 angles in both run precisions.
#include "common.cuh"

// qkv: [N, (nh + 2*nkv) * hd]; heads 0..nh-1 are q (rotated in place), the next nkv are k
// (rotated, written to the cache), the last nkv are v (copied to the cache).
// inv_freq == nullptr: no rotation (a position encoding that leaves q and k alone).
// slots[t] < 0: the token's K/V are not stored (padding rows of a fixed-shape batch).
// One block per token: the rotary_dim/2 angles are computed once and serve every head.
template <typename T>
__global__ void rope_store_kernel(T* __restrict__ qkv, const int* __restrict__ positions,
                                  const int* __restrict__ slots, const float* __restrict__ inv_freq,
                                  T* __restrict__ k_cache, T* __restrict__ v_cache, int nh, int nkv,
                                  int hd, int rotary_dim, int num_slots, int write_cache,
                                  int* status) {
    extern __shared__ float cs[];  // cos[half], sin[half]
    // Positions, slots and frequencies are inputs of the step, written before its first kernel; only the
    // q/k/v rows come from the preceding kernel.  So the angles are worked out while that one finishes.
    pdl_launch_dependents();
    const int t = blockIdx.x;
    const int half = rotary_dim >> 1;
    if (inv_freq != nullptr) {
        const float pos = (float)positions[t];
        for (int j = threadIdx.x; j < half; j += blockDim.x)
            sincosf(pos * inv_freq[j], &cs[half + j], &cs[j]);  // one argument reduction for both
    }
    int slot = slots ? slots[t] : -1;
    __syncthreads();
    pdl_wait();
    if (!write_cache) slot = -1;
    if (slot >= num_slots) {
        if (threadIdx.x == 0) cw_report(status, CW_ST_SLOT_RANGE, t, slot);
        slot = -1;
    }
    T* row0 = qkv + (size_t)t * (nh + 2 * nkv) * hd;
    // q and k heads: rotate pairs (j, j + half); k also goes to the cache
    const int rot_heads = nh + nkv;
    if (inv_freq != nullptr) {
        for (int i = threadIdx.x; i < rot_heads * half; i += blockDim.x) {
            const int head = i / half, j = i % half;
            T* row = row0 + (size_t)head * hd;
            const float c = cs[j], s = cs[half + j];
            const float x1 = to_f(row[j]), x2 = to_f(row[j + half]);
            const T o1 = from_f<T>(x1 * c - x2 * s);
            const T o2 = from_f<T>(x2 * c + x1 * s);
            row[j] = o1;  // k keeps its rotated value in the activation too
            row[j + half] = o2;
            if (head >= nh && slot >= 0) {
                T* dst = k_cache + ((size_t)slot * nkv + (head - nh)) * hd;
                dst[j] = o1;
                dst[j + half] = o2;
            }
        }
    }
    if (slot >= 0) {
        // what rotation did not touch of k (beyond the rotary span, or everything without rotation)
        const int from = inv_freq != nullptr ? rotary_dim : 0;
        const int span = hd - from;
        for (int i = threadIdx.x; i < nkv * span; i += blockDim.x) {
            const int kvh = i / span, d = from + i % span;
            k_cache[((size_t)slot * nkv + kvh) * hd + d] = row0[(size_t)(nh + kvh) * hd + d];
        }
        for (int i = threadIdx.x; i < nkv * hd; i += blockDim.x)
            v_cache[(size_t)slot * nkv * hd + i] = row0[(size_t)(nh + nkv) * hd + i];
    }
}

// The same with 16-byte accesses: a thread rotates VEC consecutive pairs (j.., j + half..) of one
// head.  Needs the head size and half the rotary span to be multiples of VEC = 16 / sizeof(T) and
// 16-byte aligned rows; the arithmetic is the scalar kernel's, element for element.
template <typename T>
struct RowVec {
    static constexpr int N = 16 / sizeof(T);
    uint4 raw;
    __device__ __forceinline__ float get(int e) const;
    __device__ __forceinline__ void set(int e, float v);
};
template <>
__device__ __forceinline__ float RowVec<float>::get(int e) const { return reinterpret_cast<const float*>(&raw)[e]; }
template <>
__device__ __forceinline__ void RowVec<float>::set(int e, float v) { reinterpret_cast<float*>(&raw)[e] = v; }
template <>
__device__ __forceinline__ float RowVec<bf16>::get(int e) const { return __bfloat162float(reinterpret_cast<const bf16*>(&raw)[e]); }
template <>
__device__ __forceinline__ void RowVec<bf16>::set(int e, float v) { reinterpret_cast<bf16*>(&raw)[e] = __float2bfloat16_rn(v); }

template <typename T>
__global__ void rope_store_vec_kernel(T* __restrict__ qkv, const int* __restrict__ positions,
                                      const int* __restrict__ slots, const float* __restrict__ inv_freq,
                                      T* __restrict__ k_cache, T* __restrict__ v_cache, int nh, int nkv,
                                      int hd, int rotary_dim, int num_slots, int write_cache, int* status) {
    constexpr int VEC = RowVec<T>::N;
    extern __shared__ float cs[];  // cos[half], sin[half]
    // Positions, slots and frequencies are inputs of the step, written before its first kernel; only the
    // q/k/v rows come from the preceding kernel.  So the angles are worked out while that one finishes.
    pdl_launch_dependents();
    const int t = blockIdx.x;
    const int half = rotary_dim >> 1;
    if (inv_freq != nullptr) {
        const float pos = (float)positions[t];
        for (int j = threadIdx.x; j < half; j += blockDim.x)
            sincosf(pos * inv_freq[j], &cs[half + j], &cs[j]);  // one argument reduction for both
    }
    int slot = slots ? slots[t] : -1;
    __syncthreads();
    pdl_wait();
    if (!write_cache) slot = -1;
    if (slot >= num_slots) {
        if (threadIdx.x == 0) cw_report(status, CW_ST_SLOT_RANGE, t, slot);
        slot = -1;
    }
    T* row0 = qkv + (size_t)t * (nh + 2 * nkv) * hd;
    if (inv_freq != nullptr) {
        const int half_v = half / VEC;
        for (int i = threadIdx.x; i < (nh + nkv) * half_v; i += blockDim.x) {
            const int head = i / half_v, j = (i % half_v) * VEC;
            T* row = row0 + (size_t)head * hd;
            RowVec<T> a, b;
            a.raw = *reinterpret_cast<const uint4*>(row + j);
            b.raw = *reinterpret_cast<const uint4*>(row + j + half);
#pragma unroll
            for (int e = 0; e < VEC; ++e) {
                const float c = cs[j + e], sn = cs[half + j + e];
                const float x1 = a.get(e), x2 = b.get(e);
                a.set(e, x1 * c - x2 * sn);
                b.set(e, x2 * c + x1 * sn);
            }
            *reinterpret_cast<uint4*>(row + j) = a.raw;  // k keeps its rotated value in the activation too
            *reinterpret_cast<uint4*>(row + j + half) = b.raw;
            if (head >= nh && slot >= 0) {
                T* dst = k_cache + ((size_t)slot * nkv + (head - nh)) * hd;
                *reinterpret_cast<uint4*>(dst + j) = a.raw;
                *reinterpret_cast<uint4*>(dst + j + half) = b.raw;
            }
        }
    }
    if (slot >= 0) {
        // what rotation did not touch of k (beyond the rotary span, or everything without rotation), and v
        const int from = inv_freq != nullptr ? rotary_dim : 0;
        const int span_v = (hd - from) / VEC;
        for (int i = threadIdx.x; i < nkv * span_v; i += blockDim.x) {
            const int kvh = i / span_v, d = from + (i % span_v) * VEC;
            *reinterpret_cast<uint4*>(k_cache + ((size_t)slot * nkv + kvh) * hd + d) =
                *reinterpret_cast<const uint4*>(row0 + (size_t)(nh + kvh) * hd + d);
        }
        for (int i = threadIdx.x; i < nkv * hd / VEC; i += blockDim.x)
            *reinterpret_cast<uint4*>(v_cache + (size_t)slot * nkv * hd + (size_t)i * VEC) =
                *reinterpret_cast<const uint4*>(row0 + (size_t)(nh + nkv) * hd + (size_t)i * VEC);
    }
}

extern "C" int cw_rope_store(void* qkv, const int* positions, const int* slots,
                             const float* inv_freq, void* k_cache, void* v_cache, int N, int nh,
                             int nkv, int hd, int rotary_dim, int num_slots, int write_cache,
                             int dtype, int* status, cudaStream_t stream) {
    if (N == 0) return CW_OK;
    if (N < 0 || nh <= 0 || nkv <= 0 || hd <= 0) return CW_ERR_BAD_SIZE;
    if (rotary_dim < 0 || rotary_dim > hd || (rotary_dim & 1)) return CW_ERR_BAD_SIZE;
    const dim3 grid(N);
    const int work = (nh + nkv) * (hd / 2);
    const int threads = work >= 1024 ? 256 : (work >= 256 ? 128 : 64);
    const size_t smem = (size_t)rotary_dim * sizeof(float);
    const int vec = dtype == 0 ? 4 : 8;
    const bool wide = hd % vec == 0 && (rotary_dim / 2) % vec == 0 && ((uintptr_t)qkv & 15) == 0 &&
                      ((uintptr_t)k_cache & 15) == 0 && ((uintptr_t)v_cache & 15) == 0;
    if (wide) {
        const int vthreads = work / vec >= 128 ? 128 : 64;
        if (dtype == 0)
            return cw_launch(rope_store_vec_kernel<float>, grid, dim3(vthreads), smem, stream, 1, (float*)qkv, positions,
                             slots, inv_freq, (float*)k_cache, (float*)v_cache, nh, nkv, hd, rotary_dim, num_slots,
                             write_cache, status);
        if (dtype == 1)
            return cw_launch(rope_store_vec_kernel<bf16>, grid, dim3(vthreads), smem, stream, 1, (bf16*)qkv, positions,
                             slots, inv_freq, (bf16*)k_cache, (bf16*)v_cache, nh, nkv, hd, rotary_dim, num_slots,
                             write_cache, status);
        return CW_ERR_BAD_DTYPE;
    }
    if (dtype == 0)
        return cw_launch(rope_store_kernel<float>, grid, dim3(threads), smem, stream, 1, (float*)qkv, positions, slots,
                         inv_freq, (float*)k_cache, (float*)v_cache, nh, nkv, hd, rotary_dim, num_slots,
                         write_cache, status);
    if (dtype == 1)
        return cw_launch(rope_store_kernel<bf16>, grid, dim3(threads), smem, stream, 1, (bf16*)qkv, positions, slots,
                         inv_freq, (bf16*)k_cache, (bf16*)v_cache, nh, nkv, hd, rotary_dim, num_slots,
                         write_cache, status);
    return CW_ERR_BAD_DTYPE;
}

// cache: [planes, num_pages, page_elems]; copies page src->dst in every plane (a plane is one
// layer's K or V).  pairs: int32 [num_pairs, 2].
__global__ void copy_pages_kernel(uint4* __restrict__ cache, const int* __restrict__ pairs,
                                  size_t page_vec, size_t plane_vec, int num_pages, int* status) {
    const int src = pairs[2 * blockIdx.x], dst = pairs[2 * blockIdx.x + 1];
    if (src < 0 || src >= num_pages || dst < 0 || dst >= num_pages) {
        if (threadIdx.x == 0) cw_report(status, CW_ST_PAGE_RANGE, src, dst);
        return;
    }
    uint4* base = cache + (size_t)blockIdx.y * plane_vec;
    for (size_t i = threadIdx.x; i < page_vec; i += blockDim.x)
        base[(size_t)dst * page_vec + i] = base[(size_t)src * page_vec + i];
}

extern "C" int cw_copy_pages(void* cache, const int* pairs, int num_pairs, int planes,
                             int num_pages, long long page_bytes, int* status,
                             cudaStream_t stream) {
    if (num_pairs == 0) return CW_OK;
    if (num_pairs < 0 || planes <= 0 || planes > 65535 || page_bytes <= 0 || page_bytes % 16)
        return CW_ERR_BAD_SIZE;
    const size_t page_vec = (size_t)page_bytes / 16;
    dim3 grid(num_pairs, planes);
    copy_pages_kernel<<<grid, 128, 0, stream>>>((uint4*)cache, pairs, page_vec,
                                                page_vec * (size_t)num_pages, num_pages, status);
    return CW_LAUNCH_CHECK();
}

CW_TRACE_TU(rope_cache)
