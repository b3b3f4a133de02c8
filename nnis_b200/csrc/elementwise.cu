// Row-wise kernels around the matrix products: embedding gather, RMSNorm,
// the gated activation, and RoPE fused with the store into the paged cache.
// The residual stream is float32 in both engine dtypes; T is the dtype of the
// matrix-product operands (float or bfloat16).  Statistics, angles and the
// activation are computed in float32 and rounded once on the store.
#include "async_copy.cuh"
#include "common.cuh"

namespace nnis {

// ---------------------------------------------------------------------------
// hidden[n, :] = table[token[n], :]  (widened exactly to float32)
// NNIS: crates/nnis-kernels/src/gather.rs:17-33.
// ---------------------------------------------------------------------------
template <typename T>
__global__ void embed_kernel(const T* __restrict__ table, const int* __restrict__ tokens,
                             float* __restrict__ hidden, int n_tokens, int width, int vocab,
                             int* __restrict__ status) {
    int n = blockIdx.x;
    int token = tokens[n];
    bool bad = token < 0 || token >= vocab;
    if (bad) {
        if (threadIdx.x == 0) atomicExch(status, 1);
        token = 0;
    }
    const T* row = table + (size_t)token * width;
    float* out = hidden + (size_t)n * width;
    for (int i = threadIdx.x; i < width; i += blockDim.x) out[i] = bad ? 0.f : to_float(row[i]);
}

// ---------------------------------------------------------------------------
// y = (x * 1/sqrt(mean(x^2) + eps)) * w, one block per output row; `rows`
// (optional) picks the input row of each output row.
// NNIS: crates/nnis-model/src/kernels.rs:15-48.
// ---------------------------------------------------------------------------
template <typename T>
__global__ void rmsnorm_kernel(const float* __restrict__ x, const int* __restrict__ rows,
                               const float* __restrict__ w, T* __restrict__ y, int width,
                               float eps) {
    __shared__ float partial[32];
    __shared__ float scale_s;
    // launched as a programmatic dependent: x comes from the kernel before this one
    pdl_wait();
    pdl_launch_dependents();
    int r = blockIdx.x;
    const float* in = x + (size_t)(rows ? rows[r] : r) * width;
    float ss = 0.f;
    for (int i = threadIdx.x; i < width; i += blockDim.x) ss = fmaf(in[i], in[i], ss);
    ss = warp_sum(ss);
    int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n_warps = blockDim.x >> 5;
    if (lane == 0) partial[warp] = ss;
    __syncthreads();
    if (warp == 0) {
        float v = lane < n_warps ? partial[lane] : 0.f;
        v = warp_sum(v);
        if (lane == 0) scale_s = 1.0f / sqrtf(v * (1.0f / (float)width) + eps);
    }
    __syncthreads();
    float s = scale_s;
    T* out = y + (size_t)r * width;
    for (int i = threadIdx.x; i < width; i += blockDim.x) out[i] = from_float<T>((in[i] * s) * w[i]);
}

// The same for many rows of moderate width (a multiple of 4, at most 1,024): a
// warp per row, the row kept in registers between the sum and the scaling, no
// barrier; eight rows per CTA.
template <typename T>
__global__ void __launch_bounds__(256)
rmsnorm_rows_kernel(const float* __restrict__ x, const int* __restrict__ rows,
                    const float* __restrict__ w, T* __restrict__ y, int n_rows, int width, float eps,
                    unsigned long long* trace) {
    trace_mark(trace, 0);
    const int lane = threadIdx.x & 31, r = blockIdx.x * 8 + (threadIdx.x >> 5);
    const float4* w4 = reinterpret_cast<const float4*>(w);
    const int n4 = width >> 2;
    // the norm's weights depend on no kernel: they are fetched before the wait
    float4 g[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        int c = lane + 32 * j;
        g[j] = c < n4 ? w4[c] : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    pdl_wait();
    pdl_launch_dependents();
    trace_mark(trace, 2);
    trace_mark(trace, 3);
    if (r >= n_rows) {
        trace_mark(trace, 1);
        return;
    }
    const float4* in = reinterpret_cast<const float4*>(x + (size_t)(rows ? rows[r] : r) * width);
    float4 v[8];
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        int c = lane + 32 * j;
        v[j] = c < n4 ? in[c] : make_float4(0.f, 0.f, 0.f, 0.f);
        ss = fmaf(v[j].x, v[j].x, ss);
        ss = fmaf(v[j].y, v[j].y, ss);
        ss = fmaf(v[j].z, v[j].z, ss);
        ss = fmaf(v[j].w, v[j].w, ss);
    }
    ss = warp_sum(ss);
    const float s = 1.0f / sqrtf(ss * (1.0f / (float)width) + eps);
    T* out = y + (size_t)r * width;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        int c = lane + 32 * j;
        if (c < n4)
            store4(out + c * 4, make_float4((v[j].x * s) * g[j].x, (v[j].y * s) * g[j].y, (v[j].z * s) * g[j].z,
                                            (v[j].w * s) * g[j].w));
    }
    trace_mark(trace, 1);
}

// ---------------------------------------------------------------------------
// out[n, i] = silu(g[n, i]) * u[n, i]; gate and up are the two halves of one
// float32 row [2 * inter].  NNIS: crates/nnis-model/src/fused_swiglu.rs:14-27.
// ---------------------------------------------------------------------------
template <typename T>
__global__ void silu_mul_kernel(const float* __restrict__ gate_up, T* __restrict__ out,
                                size_t n_rows, int inter) {
    size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= n_rows * (size_t)inter) return;
    size_t n = idx / inter;
    int i = (int)(idx - n * inter);
    float g = gate_up[n * 2 * inter + i];
    float u = gate_up[n * 2 * inter + inter + i];
    out[idx] = from_float<T>((g / (1.0f + expf(-g))) * u);
}

// ---------------------------------------------------------------------------
// Rotate-half RoPE on the q and k heads of a packed [n, (nq + 2 nkv) * d] row,
// in place, and store rotated k and plain v at each token's position of the
// paged cache.  cos/sin: [max_positions, d/2] float32.  With `rotate == 0` only
// the store happens; with nkv == 0 only q is rotated (a layer that reads another
// layer's cache).
// NNIS: crates/nnis-model/src/runtime_kernels.rs:38-66 and the append in
// crates/nnis-rt/src/kv_cache.rs:212-366.
// ---------------------------------------------------------------------------
template <typename T>
__global__ void rope_store_kernel(T* __restrict__ qkv, const int* __restrict__ token_pos,
                                  const int* __restrict__ token_seq,
                                  const int* __restrict__ page_table, int table_cols,
                                  const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                                  T* __restrict__ k_cache, T* __restrict__ v_cache, int nq, int nkv,
                                  int d, int page_size, int rotate) {
    int n = blockIdx.x;
    int pos = token_pos[n];
    if (pos < 0) return;  // a padding row: nothing to rotate, nothing to store
    int half = d >> 1;
    T* row = qkv + (size_t)n * (nq + 2 * nkv) * d;
    size_t page_base = 0;
    int in_page = 0;
    if (nkv > 0) {
        int page = page_table[(size_t)token_seq[n] * table_cols + pos / page_size];
        page_base = (size_t)page * nkv * page_size * d;
        in_page = pos % page_size;
    }
    int rot_items = (nq + nkv) * half;
    for (int it = threadIdx.x; it < rot_items; it += blockDim.x) {
        int head = it / half, j = it - head * half;
        T* h = row + (size_t)head * d;
        float a = to_float(h[j]), b = to_float(h[j + half]);
        float ra = a, rb = b;
        if (rotate) {
            float c = cos_t[(size_t)pos * half + j], s = sin_t[(size_t)pos * half + j];
            ra = a * c - b * s;
            rb = b * c + a * s;
        }
        T ta = from_float<T>(ra), tb = from_float<T>(rb);
        h[j] = ta;
        h[j + half] = tb;
        if (head >= nq) {
            size_t dst = page_base + ((size_t)(head - nq) * page_size + in_page) * d;
            k_cache[dst + j] = ta;
            k_cache[dst + j + half] = tb;
        }
    }
    const T* vrow = row + (size_t)(nq + nkv) * d;
    for (int it = threadIdx.x; it < nkv * d; it += blockDim.x) {
        int head = it / d, i = it - head * d;
        v_cache[page_base + ((size_t)head * page_size + in_page) * d + i] = vrow[it];
    }
}

}  // namespace nnis

using namespace nnis;

// A copy in either direction on the stream (pinned host memory on the host side),
// for the few bytes a decode step exchanges with the host: one call, no allocation.
NNIS_API int nnis_copy_async(void* dst, const void* src, long long bytes, cudaStream_t stream) {
    if (!dst || !src || bytes <= 0) return NNIS_ERR_ARGUMENT;
    cudaError_t e = cudaMemcpyAsync(dst, src, (size_t)bytes, cudaMemcpyDefault, stream);
    return e == cudaSuccess ? NNIS_OK : (int)e;
}

NNIS_API int nnis_stream_synchronize(cudaStream_t stream) {
    cudaError_t e = cudaStreamSynchronize(stream);
    return e == cudaSuccess ? NNIS_OK : (int)e;
}

NNIS_API int nnis_embed(const void* table, int dtype, const int* tokens, float* hidden,
                        int n_tokens, int width, int vocab, int* status, cudaStream_t stream) {
    if (n_tokens <= 0 || width <= 0 || vocab <= 0 || !status) return NNIS_ERR_ARGUMENT;
    int threads = width >= 256 ? 256 : 64;
    if (dtype == NNIS_DTYPE_F32)
        embed_kernel<float><<<n_tokens, threads, 0, stream>>>((const float*)table, tokens, hidden,
                                                              n_tokens, width, vocab, status);
    else if (dtype == NNIS_DTYPE_BF16)
        embed_kernel<bf16><<<n_tokens, threads, 0, stream>>>((const bf16*)table, tokens, hidden,
                                                             n_tokens, width, vocab, status);
    else
        return NNIS_ERR_UNSUPPORTED;
    NNIS_RETURN_LAUNCH();
}

// `pdl`: launch as a programmatic dependent of the kernel before it on the stream
// (the kernel waits for that kernel's results itself).
NNIS_API int nnis_rmsnorm(const float* x, const int* rows, const float* w, void* y, int out_dtype,
                          int n_rows, int width, float eps, int pdl, cudaStream_t stream) {
    if (n_rows <= 0 || width <= 0 || !(eps > 0.f)) return NNIS_ERR_ARGUMENT;
    // many rows of moderate width on 16-byte boundaries: a warp per row
    const bool by_rows = n_rows >= 64 && width % 4 == 0 && width <= 1024 &&
                         ((uintptr_t)x | (uintptr_t)w | (uintptr_t)y) % 16 == 0;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(by_rows ? (n_rows + 7) / 8 : n_rows);
    cfg.blockDim = dim3(by_rows ? 256 : (width >= 1024 ? 256 : (width >= 256 ? 128 : 32)));
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 1 : 0;
    cudaError_t e;
    if (out_dtype == NNIS_DTYPE_F32)
        e = by_rows ? cudaLaunchKernelEx(&cfg, rmsnorm_rows_kernel<float>, x, rows, w, (float*)y, n_rows, width, eps, trace_slot("rmsnorm rows"))
                    : cudaLaunchKernelEx(&cfg, rmsnorm_kernel<float>, x, rows, w, (float*)y, width, eps);
    else if (out_dtype == NNIS_DTYPE_BF16)
        e = by_rows ? cudaLaunchKernelEx(&cfg, rmsnorm_rows_kernel<bf16>, x, rows, w, (bf16*)y, n_rows, width, eps, trace_slot("rmsnorm rows"))
                    : cudaLaunchKernelEx(&cfg, rmsnorm_kernel<bf16>, x, rows, w, (bf16*)y, width, eps);
    else
        return NNIS_ERR_UNSUPPORTED;
    return e == cudaSuccess ? NNIS_OK : (int)e;
}

NNIS_API int nnis_silu_mul(const float* gate_up, void* out, int out_dtype, long long n_rows,
                           int inter, cudaStream_t stream) {
    if (n_rows <= 0 || inter <= 0) return NNIS_ERR_ARGUMENT;
    size_t total = (size_t)n_rows * inter;
    unsigned blocks = (unsigned)((total + 255) / 256);
    if (out_dtype == NNIS_DTYPE_F32)
        silu_mul_kernel<float><<<blocks, 256, 0, stream>>>(gate_up, (float*)out, n_rows, inter);
    else if (out_dtype == NNIS_DTYPE_BF16)
        silu_mul_kernel<bf16><<<blocks, 256, 0, stream>>>(gate_up, (bf16*)out, n_rows, inter);
    else
        return NNIS_ERR_UNSUPPORTED;
    NNIS_RETURN_LAUNCH();
}

NNIS_API int nnis_rope_store(void* qkv, int dtype, const int* token_pos, const int* token_seq,
                             const int* page_table, int table_cols, const float* cos_t,
                             const float* sin_t, void* k_cache, void* v_cache, int n_tokens, int nq,
                             int nkv, int d, int page_size, int rotate, cudaStream_t stream) {
    if (n_tokens <= 0 || nq < 0 || nkv < 0 || nq + nkv == 0 || d <= 0 || (d & 1))
        return NNIS_ERR_ARGUMENT;
    if (nkv > 0 && (!page_table || !k_cache || !v_cache || page_size <= 0 || table_cols <= 0))
        return NNIS_ERR_ARGUMENT;
    if (rotate && (!cos_t || !sin_t)) return NNIS_ERR_ARGUMENT;
    int work = (nq + nkv) * (d / 2);
    int threads = work >= 256 ? 256 : (work >= 128 ? 128 : 64);
    if (dtype == NNIS_DTYPE_F32)
        rope_store_kernel<float><<<n_tokens, threads, 0, stream>>>(
            (float*)qkv, token_pos, token_seq, page_table, table_cols, cos_t, sin_t,
            (float*)k_cache, (float*)v_cache, nq, nkv, d, page_size, rotate);
    else if (dtype == NNIS_DTYPE_BF16)
        rope_store_kernel<bf16><<<n_tokens, threads, 0, stream>>>(
            (bf16*)qkv, token_pos, token_seq, page_table, table_cols, cos_t, sin_t, (bf16*)k_cache,
            (bf16*)v_cache, nq, nkv, d, page_size, rotate);
    else
        return NNIS_ERR_UNSUPPORTED;
    NNIS_RETURN_LAUNCH();
}
