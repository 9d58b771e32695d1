// Plain tiled matrix product on the CUDA cores with float32 accumulation:
//   C[M,N] = A[M,K] * W[N,K]^T (+ bias[N]),   W in nn.Linear layout (clockwork/engine/model.py:58-60, 74-77)
// It is the matrix product of the true-float32 path (fmaf only, no tensor cores, no TF32) and
// the fallback of the bfloat16 path for sizes the tensor-core kernel refuses.
// Every output element is summed in the same fixed order whatever M, N or the tile it falls in, so
// a row's result does not depend on the rest of the batch: fmaf chains over 16 consecutive k, in
// ascending order, whose results are added up with a compensated (Kahan) running sum.  One plain
// chain over a long inner dimension would lose more than the 1e-5 that the float32 path is held
// to: at K = 8960 its rounding error alone is of that order; summed this way the result stays
// within a few units in the last place of the exact dot product at any K.
//
// Epilogues: 0 store as T; 1 add into a float32 matrix (the residual stream); 2 store float32
// (logits).  The SwiGLU variant computes silu(A Wg^T) * (A Wu^T) (clockwork/engine/model.py:62-63).
#include "common.cuh"

#define BM 64
#define BN 64
#define BK 16

// sum += x with the rounding error of earlier additions carried along in `lost` (Kahan's summation;
// the order of the operations matters and the compiler keeps it: no fast-math flags are used)
__device__ __forceinline__ void kahan_add(float& sum, float& lost, float x) {
    const float y = __fsub_rn(x, lost);
    const float t = __fadd_rn(sum, y);
    lost = __fsub_rn(__fsub_rn(t, sum), y);
    sum = t;
}

template <typename T, bool SWIGLU>
__global__ void __launch_bounds__(256)
gemm_ref_kernel(const T* __restrict__ A, const T* __restrict__ W, const T* __restrict__ W2,
                const float* __restrict__ bias, void* __restrict__ Cout, int M, int N, int K,
                int lda, int ldc, int epilogue) {
    __shared__ float As[BK][BM + 4];
    __shared__ float Ws[BK][BN + 4];
    __shared__ float W2s[SWIGLU ? BK : 1][BN + 4];
    const int tid = threadIdx.x;
    const int tx = tid & 15, ty = tid >> 4;
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    float sum[4][4] = {}, lost[4][4] = {};    // running sums and what their roundings have lost so far
    float sum2[4][4] = {}, lost2[4][4] = {};
    for (int k0 = 0; k0 < K; k0 += BK) {
        float acc[4][4] = {};
        float acc2[4][4] = {};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int e = tid + i * 256;      // 0..1023
            const int r = e >> 4, c = e & 15; // row in tile, k in tile
            const int k = k0 + c;
            float a = 0.f, w = 0.f, w2 = 0.f;
            if (k < K) {
                if (m0 + r < M) a = to_f(A[(size_t)(m0 + r) * lda + k]);
                if (n0 + r < N) {
                    w = to_f(W[(size_t)(n0 + r) * K + k]);
                    if (SWIGLU) w2 = to_f(W2[(size_t)(n0 + r) * K + k]);
                }
            }
            As[c][r] = a;
            Ws[c][r] = w;
            if (SWIGLU) W2s[c][r] = w2;
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < BK; ++k) {
            float a[4], w[4], w2[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = As[k][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) w[j] = Ws[k][tx * 4 + j];
            if (SWIGLU) {
#pragma unroll
                for (int j = 0; j < 4; ++j) w2[j] = W2s[k][tx * 4 + j];
            }
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
                    if (SWIGLU) acc2[i][j] = fmaf(a[i], w2[j], acc2[i][j]);
                }
        }
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                kahan_add(sum[i][j], lost[i][j], acc[i][j]);
                if (SWIGLU) kahan_add(sum2[i][j], lost2[i][j], acc2[i][j]);
            }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int m = m0 + ty * 4 + i;
        if (m >= M) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int n = n0 + tx * 4 + j;
            if (n >= N) continue;
            float v = sum[i][j];
            if (bias) v += bias[n];
            const size_t idx = (size_t)m * ldc + n;
            if (SWIGLU) {
                const float g = v, u = sum2[i][j];
                ((T*)Cout)[idx] = from_f<T>(g / (1.0f + expf(-g)) * u);
            } else if (epilogue == 0) {
                ((T*)Cout)[idx] = from_f<T>(v);
            } else if (epilogue == 1) {
                ((float*)Cout)[idx] += v;
            } else {
                ((float*)Cout)[idx] = v;
            }
        }
    }
}

extern "C" int cw_gemm_ref(const void* A, const void* W, const float* bias, void* C, int M, int N,
                           int K, int lda, int ldc, int epilogue, int dtype,
                           cudaStream_t stream) {
    if (M == 0 || N == 0) return CW_OK;
    if (M < 0 || N < 0 || K <= 0 || lda < K || ldc < N) return CW_ERR_BAD_SIZE;
    if (epilogue < 0 || epilogue > 2) return CW_ERR_UNSUPPORTED;
    dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
    if (grid.y > 65535) return CW_ERR_BAD_SIZE;
    if (dtype == 0)
        gemm_ref_kernel<float, false><<<grid, 256, 0, stream>>>(
            (const float*)A, (const float*)W, nullptr, bias, C, M, N, K, lda, ldc, epilogue);
    else if (dtype == 1)
        gemm_ref_kernel<bf16, false><<<grid, 256, 0, stream>>>(
            (const bf16*)A, (const bf16*)W, nullptr, bias, C, M, N, K, lda, ldc, epilogue);
    else
        return CW_ERR_BAD_DTYPE;
    return CW_LAUNCH_CHECK();
}

extern "C" int cw_gemm_ref_swiglu(const void* A, const void* Wgate, const void* Wup, void* C,
                                  int M, int N, int K, int dtype, cudaStream_t stream) {
    if (M == 0 || N == 0) return CW_OK;
    if (M < 0 || N < 0 || K <= 0) return CW_ERR_BAD_SIZE;
    dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
    if (grid.y > 65535) return CW_ERR_BAD_SIZE;
    if (dtype == 0)
        gemm_ref_kernel<float, true><<<grid, 256, 0, stream>>>(
            (const float*)A, (const float*)Wgate, (const float*)Wup, nullptr, C, M, N, K, K, N, 0);
    else if (dtype == 1)
        gemm_ref_kernel<bf16, true><<<grid, 256, 0, stream>>>(
            (const bf16*)A, (const bf16*)Wgate, (const bf16*)Wup, nullptr, C, M, N, K, K, N, 0);
    else
        return CW_ERR_BAD_DTYPE;
    return CW_LAUNCH_CHECK();
}

CW_TRACE_TU(gemm_ref)
