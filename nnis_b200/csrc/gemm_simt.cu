// Matrix products on the CUDA cores: C[M,N] (op)= A[M,K] . W[N,K]^T + bias.
// W is stored [out, in] row-major as the checkpoint has it, so both operands
// run along K.  Operands are float32 or bfloat16; products are accumulated in
// float32 with fmaf, never through a reduced-precision tensor-core mode.  These
// are the whole float32 path, and the fallback of the bfloat16 path for shapes
// that the tcgen05 kernel refuses.
//
// Output modes: 0 store in the operand dtype, 1 store float32, 2 add to a
// float32 destination (the residual stream).
// NNIS: crates/nnis-kernels/src/gemm.rs:16-64 (tiled product),
// crates/nnis-kernels/src/gemv.rs:45-61 (one-token projection).
#include "common.cuh"

namespace nnis {

template <typename T, int MODE>
__device__ __forceinline__ void emit(void* C, size_t idx, float v) {
    if (MODE == 0) reinterpret_cast<T*>(C)[idx] = from_float<T>(v);
    else if (MODE == 1) reinterpret_cast<float*>(C)[idx] = v;
    else reinterpret_cast<float*>(C)[idx] += v;
}

// ---- 64 x 64 tile, 16 deep, 256 threads, 4 x 4 outputs per thread -----------
template <typename T, int MODE, bool VEC>
__global__ void __launch_bounds__(256)
gemm_tile_kernel(const T* __restrict__ A, const T* __restrict__ W, const float* __restrict__ bias,
                 void* __restrict__ C, int M, int N, int K) {
    constexpr int BM = 64, BN = 64, BK = 16, PAD = 4;
    __shared__ __align__(16) float As[BK][BM + PAD];
    __shared__ __align__(16) float Ws[BK][BN + PAD];
    int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
    int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    int lr = tid >> 2, lk = (tid & 3) * 4;
    float acc[4][4] = {};
    for (int k0 = 0; k0 < K; k0 += BK) {
        float a[4] = {0.f, 0.f, 0.f, 0.f}, w[4] = {0.f, 0.f, 0.f, 0.f};
        int gk = k0 + lk;
        if (VEC) {
            if (m0 + lr < M && gk < K) {
                float4 v = load4(A + (size_t)(m0 + lr) * K + gk);
                a[0] = v.x; a[1] = v.y; a[2] = v.z; a[3] = v.w;
            }
            if (n0 + lr < N && gk < K) {
                float4 v = load4(W + (size_t)(n0 + lr) * K + gk);
                w[0] = v.x; w[1] = v.y; w[2] = v.z; w[3] = v.w;
            }
        } else {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                if (m0 + lr < M && gk + i < K) a[i] = to_float(A[(size_t)(m0 + lr) * K + gk + i]);
                if (n0 + lr < N && gk + i < K) w[i] = to_float(W[(size_t)(n0 + lr) * K + gk + i]);
            }
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            As[lk + i][lr] = a[i];
            Ws[lk + i][lr] = w[i];
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < BK; ++k) {
            float4 av = *reinterpret_cast<const float4*>(&As[k][ty * 4]);
            float4 wv = *reinterpret_cast<const float4*>(&Ws[k][tx * 4]);
            float ar[4] = {av.x, av.y, av.z, av.w}, wr[4] = {wv.x, wv.y, wv.z, wv.w};
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(ar[i], wr[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        int m = m0 + ty * 4 + i;
        if (m >= M) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            int n = n0 + tx * 4 + j;
            if (n >= N) continue;
            float v = acc[i][j] + (bias ? bias[n] : 0.f);
            emit<T, MODE>(C, (size_t)m * N + n, v);
        }
    }
}

// ---- few rows (decoding): one warp per output column, MT rows at a time -----
template <typename T, int MT, int MODE, bool VEC>
__global__ void __launch_bounds__(256)
gemm_rows_kernel(const T* __restrict__ A, const T* __restrict__ W, const float* __restrict__ bias,
                 void* __restrict__ C, int M, int N, int K) {
    int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    int n = blockIdx.x * 8 + warp;
    int m0 = blockIdx.y * MT;
    if (n >= N) return;
    float acc[MT];
#pragma unroll
    for (int i = 0; i < MT; ++i) acc[i] = 0.f;
    const T* wrow = W + (size_t)n * K;
    if (VEC) {
        for (int k = lane * 4; k < K; k += 128) {
            float4 w = load4(wrow + k);
#pragma unroll
            for (int i = 0; i < MT; ++i) {
                if (m0 + i < M) {
                    float4 a = load4(A + (size_t)(m0 + i) * K + k);
                    acc[i] = fmaf(a.x, w.x, acc[i]);
                    acc[i] = fmaf(a.y, w.y, acc[i]);
                    acc[i] = fmaf(a.z, w.z, acc[i]);
                    acc[i] = fmaf(a.w, w.w, acc[i]);
                }
            }
        }
    } else {
        for (int k = lane; k < K; k += 32) {
            float w = to_float(wrow[k]);
#pragma unroll
            for (int i = 0; i < MT; ++i)
                if (m0 + i < M) acc[i] = fmaf(to_float(A[(size_t)(m0 + i) * K + k]), w, acc[i]);
        }
    }
#pragma unroll
    for (int i = 0; i < MT; ++i) {
        float v = warp_sum(acc[i]);
        if (lane == 0 && m0 + i < M)
            emit<T, MODE>(C, (size_t)(m0 + i) * N + n, v + (bias ? bias[n] : 0.f));
    }
}

template <typename T, int MODE, bool VEC>
static int launch_mode(const T* A, const T* W, const float* bias, void* C, int M, int N, int K,
                       cudaStream_t stream) {
    if (M <= 16) {
        dim3 grid((N + 7) / 8, 1);
        if (M == 1) gemm_rows_kernel<T, 1, MODE, VEC><<<grid, 256, 0, stream>>>(A, W, bias, C, M, N, K);
        else if (M == 2) gemm_rows_kernel<T, 2, MODE, VEC><<<grid, 256, 0, stream>>>(A, W, bias, C, M, N, K);
        else if (M <= 4) gemm_rows_kernel<T, 4, MODE, VEC><<<grid, 256, 0, stream>>>(A, W, bias, C, M, N, K);
        else {
            grid.y = (M + 7) / 8;
            gemm_rows_kernel<T, 8, MODE, VEC><<<grid, 256, 0, stream>>>(A, W, bias, C, M, N, K);
        }
    } else {
        dim3 grid((N + 63) / 64, (M + 63) / 64);
        if (grid.y > 65535u) return NNIS_ERR_UNSUPPORTED;
        gemm_tile_kernel<T, MODE, VEC><<<grid, 256, 0, stream>>>(A, W, bias, C, M, N, K);
    }
    NNIS_RETURN_LAUNCH();
}

template <typename T>
static int launch_type(const void* A, const void* W, const float* bias, void* C, int M, int N, int K,
                       int mode, cudaStream_t stream) {
    const T* a = (const T*)A;
    const T* w = (const T*)W;
    bool vec = (K % 4 == 0) && ((uintptr_t)A % 16 == 0) && ((uintptr_t)W % 16 == 0);
#define NNIS_GEMM_CASE(MODE) \
    return vec ? launch_mode<T, MODE, true>(a, w, bias, C, M, N, K, stream) \
               : launch_mode<T, MODE, false>(a, w, bias, C, M, N, K, stream)
    switch (mode) {
        case 0: NNIS_GEMM_CASE(0);
        case 1: NNIS_GEMM_CASE(1);
        case 2: NNIS_GEMM_CASE(2);
        default: return NNIS_ERR_ARGUMENT;
    }
#undef NNIS_GEMM_CASE
}

}  // namespace nnis

NNIS_API int nnis_gemm_simt(const void* A, const void* W, const float* bias, void* C, int M, int N,
                            int K, int dtype, int mode, cudaStream_t stream) {
    if (M <= 0 || N <= 0 || K <= 0 || !A || !W || !C) return NNIS_ERR_ARGUMENT;
    if (dtype == NNIS_DTYPE_F32) return nnis::launch_type<float>(A, W, bias, C, M, N, K, mode, stream);
    if (dtype == NNIS_DTYPE_BF16) return nnis::launch_type<nnis::bf16>(A, W, bias, C, M, N, K, mode, stream);
    return NNIS_ERR_UNSUPPORTED;
}
