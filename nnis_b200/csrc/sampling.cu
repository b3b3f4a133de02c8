// Picking the next token on the device: greedy argmax and seeded temperature
// sampling, one block per row of float32 logits.
//
// Greedy: larger wins, ties go to the lower index
// (NNIS: crates/nnis-kernels/src/top_k.rs:57-70).
// Temperature: weights exp((x - max) / T) in float64, one SplitMix64 draw per
// row from a per-row state that the kernel advances, inverse CDF in token-id
// order.  The generator is NNIS's (crates/nnis-model/src/sampling.rs:261-284);
// its host sampler walks candidates in descending-logit order instead, so the
// two pick different tokens from the same distribution.  Top-k and top-p stay
// on the host sampler.
#include <float.h>

#include "common.cuh"

namespace nnis {

__global__ void __launch_bounds__(256)
argmax_kernel(const float* __restrict__ logits, int* __restrict__ out, int vocab) {
    __shared__ float best_v[256];
    __shared__ int best_i[256];
    const float* row = logits + (size_t)blockIdx.x * vocab;
    float bv = -FLT_MAX;
    int bi = 0x7fffffff;
    for (int i = threadIdx.x; i < vocab; i += 256) {
        float v = row[i];
        if (v > bv || bi == 0x7fffffff) { bv = v; bi = i; }
    }
    best_v[threadIdx.x] = bv;
    best_i[threadIdx.x] = bi;
    __syncthreads();
    for (int s = 128; s > 0; s >>= 1) {
        if (threadIdx.x < s) {
            float ov = best_v[threadIdx.x + s];
            int oi = best_i[threadIdx.x + s];
            float mv = best_v[threadIdx.x];
            int mi = best_i[threadIdx.x];
            if (oi != 0x7fffffff && (mi == 0x7fffffff || ov > mv || (ov == mv && oi < mi))) {
                best_v[threadIdx.x] = ov;
                best_i[threadIdx.x] = oi;
            }
        }
        __syncthreads();
    }
    if (threadIdx.x == 0) out[blockIdx.x] = best_i[0];
}

__device__ __forceinline__ unsigned long long splitmix64_next(unsigned long long* state) {
    unsigned long long z = (*state += 0x9E3779B97F4A7C15ull);
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}

__global__ void __launch_bounds__(256)
sample_temperature_kernel(const float* __restrict__ logits, const float* __restrict__ temperature,
                          unsigned long long* __restrict__ rng_state, int* __restrict__ out,
                          int vocab) {
    __shared__ double sums[256];
    __shared__ float red[256];
    __shared__ double target_s;
    __shared__ int pick_s;
    const float* row = logits + (size_t)blockIdx.x * vocab;
    int tid = threadIdx.x;
    float mx = -FLT_MAX;
    for (int i = tid; i < vocab; i += 256) mx = fmaxf(mx, row[i]);
    red[tid] = mx;
    __syncthreads();
    for (int s = 128; s > 0; s >>= 1) {
        if (tid < s) red[tid] = fmaxf(red[tid], red[tid + s]);
        __syncthreads();
    }
    mx = red[0];
    double inv_t = 1.0 / (double)temperature[blockIdx.x];
    // each thread owns one contiguous run of ids, so prefix sums follow id order
    int chunk = (vocab + 255) / 256;
    int begin = min(vocab, tid * chunk), end = min(vocab, begin + chunk);
    double mine = 0.0;
    for (int i = begin; i < end; ++i) mine += exp(((double)row[i] - (double)mx) * inv_t);
    sums[tid] = mine;
    if (tid == 0) pick_s = vocab - 1;
    __syncthreads();
    if (tid == 0) {
        double total = 0.0;
        for (int t = 0; t < 256; ++t) {
            double s = sums[t];
            sums[t] = total;  // exclusive prefix
            total += s;
        }
        unsigned long long bits = splitmix64_next(&rng_state[blockIdx.x]) >> 11;
        target_s = ((double)bits * (1.0 / 9007199254740992.0)) * total;
    }
    __syncthreads();
    double target = target_s;
    double before = sums[tid];
    if (begin < end && target >= before && (target < before + mine || tid == 255 || end == vocab)) {
        double cum = before;
        int pick = end - 1;
        for (int i = begin; i < end; ++i) {
            cum += exp(((double)row[i] - (double)mx) * inv_t);
            if (target < cum) { pick = i; break; }
        }
        pick_s = pick;
    }
    __syncthreads();
    if (tid == 0) out[blockIdx.x] = pick_s;
}

// After a decode step on the device: the picked token becomes the next input
// and live rows (position >= 0) move on by one.
__global__ void advance_kernel(int* __restrict__ tokens, int* __restrict__ pos,
                               const int* __restrict__ picked, int n) {
    int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n || pos[i] < 0) return;
    tokens[i] = picked[i];
    pos[i] += 1;
}

}  // namespace nnis

NNIS_API int nnis_advance(int* tokens, int* pos, const int* picked, int n, cudaStream_t stream) {
    if (n <= 0) return NNIS_ERR_ARGUMENT;
    nnis::advance_kernel<<<(n + 127) / 128, 128, 0, stream>>>(tokens, pos, picked, n);
    NNIS_RETURN_LAUNCH();
}

NNIS_API int nnis_argmax(const float* logits, int* out, int n_rows, int vocab, cudaStream_t stream) {
    if (n_rows <= 0 || vocab <= 0) return NNIS_ERR_ARGUMENT;
    nnis::argmax_kernel<<<n_rows, 256, 0, stream>>>(logits, out, vocab);
    NNIS_RETURN_LAUNCH();
}

NNIS_API int nnis_sample_temperature(const float* logits, const float* temperature,
                                     unsigned long long* rng_state, int* out, int n_rows, int vocab,
                                     cudaStream_t stream) {
    if (n_rows <= 0 || vocab <= 0 || !temperature || !rng_state) return NNIS_ERR_ARGUMENT;
    nnis::sample_temperature_kernel<<<n_rows, 256, 0, stream>>>(logits, temperature, rng_state, out,
                                                               vocab);
    NNIS_RETURN_LAUNCH();
}
