// Attention over the paged cache for any even head size up to 256 (NNIS asks for
// an even one and no more: crates/nnis-model/src/config.rs:38-105), any number of
// heads and groups, with an optional window: one warp per (query
// token, query head) walks the visible keys 32 at a time with an online softmax
// in float32.  It serves prompts and single decoded tokens alike, in float32 and
// in bfloat16 storage; the key range may be split over several warps whose
// partial results a second kernel merges in a fixed order.
//
// A query at position p of its sequence sees the keys lo..p of that sequence's
// pages, lo = max(0, p - window + 1) with a window, else 0.  Its own key and
// value are in the cache already (the RoPE kernel stores them first), so the
// causal rule needs no mask beyond the range.
// NNIS: crates/nnis-model/src/kernels.rs:66-125 (one query, serial keys).
#include <float.h>

#include "common.cuh"

namespace nnis {

// partial record per (token, head, split): [0] running max, [1] running sum,
// [2 .. 2+d) unnormalised output
template <typename T, int R>
__global__ void __launch_bounds__(128)
attn_warp_kernel(const T* __restrict__ q, int q_stride, const T* __restrict__ k_cache,
                 const T* __restrict__ v_cache, const int* __restrict__ token_pos,
                 const int* __restrict__ token_seq, const int* __restrict__ page_table,
                 int table_cols, T* __restrict__ out, float* __restrict__ partial, int n_tokens,
                 int nq, int nkv, int d, int page_size, int window, float scale, int n_splits) {
    extern __shared__ float q_smem[];
    int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    int n = blockIdx.x * 4 + warp;
    if (n >= n_tokens) return;
    int hq = blockIdx.y, split = blockIdx.z;
    int hk = hq / (nq / nkv);
    int pos = token_pos[n];
    float* qs = q_smem + warp * d;

    float m = -FLT_MAX, l = 0.f;
    float acc[R];
#pragma unroll
    for (int r = 0; r < R; ++r) acc[r] = 0.f;

    if (pos >= 0) {
        const T* qrow = q + (size_t)n * q_stride + (size_t)hq * d;
        for (int i = lane; i < d; i += 32) qs[i] = to_float(qrow[i]);
        __syncwarp();
        int lo = window > 0 ? max(0, pos - window + 1) : 0;
        int hi = pos + 1;
        int per = (hi - lo + n_splits - 1) / n_splits;
        per = (per + 31) & ~31;
        int start = lo + split * per;
        int end = min(hi, start + per);
        const int* table = page_table + (size_t)token_seq[n] * table_cols;
        for (int c = start; c < end; c += 32) {
            int t = c + lane;
            bool valid = t < end;
            int row_index = 0;
            float s = -FLT_MAX;
            if (valid) {
                int page = table[t / page_size];
                row_index = (page * nkv + hk) * page_size + (t % page_size);
                const T* krow = k_cache + (size_t)row_index * d;
                float dot = 0.f;
                const int d4 = (d & 3) ? 0 : d;  // rows of a head size that is no multiple of
                for (int i = 0; i < d4; i += 4) {  // four start on 8- or 4-byte boundaries only
                    float4 kv = load4(krow + i);
                    dot = fmaf(qs[i], kv.x, dot);
                    dot = fmaf(qs[i + 1], kv.y, dot);
                    dot = fmaf(qs[i + 2], kv.z, dot);
                    dot = fmaf(qs[i + 3], kv.w, dot);
                }
                for (int i = d4; i < d; i += 2) {
                    float2 kv = load2(krow + i);
                    dot = fmaf(qs[i], kv.x, dot);
                    dot = fmaf(qs[i + 1], kv.y, dot);
                }
                s = dot * scale;
            }
            float m_new = fmaxf(m, warp_max(s));
            float p = valid ? expf(s - m_new) : 0.f;
            float alpha = l == 0.f ? 0.f : expf(m - m_new);
            l = l * alpha + warp_sum(p);
            m = m_new;
#pragma unroll
            for (int r = 0; r < R; ++r) acc[r] *= alpha;
            int count = min(32, end - c);
            for (int j = 0; j < count; ++j) {
                float pj = __shfl_sync(0xffffffffu, p, j);
                int rj = __shfl_sync(0xffffffffu, row_index, j);
                const T* vrow = v_cache + (size_t)rj * d;
#pragma unroll
                for (int r = 0; r < R; ++r) {
                    int i = lane + 32 * r;
                    if (i < d) acc[r] = fmaf(pj, to_float(vrow[i]), acc[r]);
                }
            }
        }
    }
    if (n_splits == 1) {
        float inv = l > 0.f ? 1.0f / l : 0.f;
        T* o = out + ((size_t)n * nq + hq) * d;
#pragma unroll
        for (int r = 0; r < R; ++r) {
            int i = lane + 32 * r;
            if (i < d) o[i] = from_float<T>(acc[r] * inv);
        }
    } else {
        float* rec = partial + (((size_t)n * nq + hq) * n_splits + split) * (size_t)(d + 2);
        if (lane == 0) {
            rec[0] = m;
            rec[1] = l;
        }
#pragma unroll
        for (int r = 0; r < R; ++r) {
            int i = lane + 32 * r;
            if (i < d) rec[2 + i] = acc[r];
        }
    }
}

// Merge the splits of one (token, head) in ascending order of split.
template <typename T>
__global__ void attn_merge_kernel(const float* __restrict__ partial, T* __restrict__ out,
                                  size_t n_rows, int d, int n_splits) {
    size_t row = (size_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    int lane = threadIdx.x & 31;
    if (row >= n_rows) return;
    const float* rec = partial + row * n_splits * (size_t)(d + 2);
    float m = -FLT_MAX;
    for (int s = 0; s < n_splits; ++s)
        if (rec[(size_t)s * (d + 2) + 1] > 0.f) m = fmaxf(m, rec[(size_t)s * (d + 2)]);
    float l = 0.f;
    for (int s = 0; s < n_splits; ++s) {
        float ls = rec[(size_t)s * (d + 2) + 1];
        if (ls > 0.f) l += ls * expf(rec[(size_t)s * (d + 2)] - m);
    }
    float inv = l > 0.f ? 1.0f / l : 0.f;
    for (int i = lane; i < d; i += 32) {
        float o = 0.f;
        for (int s = 0; s < n_splits; ++s) {
            float ls = rec[(size_t)s * (d + 2) + 1];
            if (ls > 0.f) o += rec[(size_t)s * (d + 2) + 2 + i] * expf(rec[(size_t)s * (d + 2)] - m);
        }
        out[row * d + i] = from_float<T>(o * inv);
    }
}

template <typename T>
static int launch_attention(const void* q, int q_stride, const void* k_cache, const void* v_cache,
                            const int* token_pos, const int* token_seq, const int* page_table,
                            int table_cols, void* out, float* partial, int n_tokens, int nq,
                            int nkv, int d, int page_size, int window, float scale, int n_splits,
                            cudaStream_t stream) {
    dim3 grid((n_tokens + 3) / 4, nq, n_splits);
    size_t smem = 4 * (size_t)d * sizeof(float);
#define NNIS_ATTN_CASE(R) \
    attn_warp_kernel<T, R><<<grid, 128, smem, stream>>>( \
        (const T*)q, q_stride, (const T*)k_cache, (const T*)v_cache, token_pos, token_seq, \
        page_table, table_cols, (T*)out, partial, n_tokens, nq, nkv, d, page_size, window, scale, \
        n_splits)
    if (d <= 32) NNIS_ATTN_CASE(1);
    else if (d <= 64) NNIS_ATTN_CASE(2);
    else if (d <= 128) NNIS_ATTN_CASE(4);
    else NNIS_ATTN_CASE(8);
#undef NNIS_ATTN_CASE
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return (int)e;
    if (n_splits > 1) {
        size_t rows = (size_t)n_tokens * nq;
        attn_merge_kernel<T><<<(unsigned)((rows + 3) / 4), 128, 0, stream>>>(partial, (T*)out, rows,
                                                                             d, n_splits);
    }
    NNIS_RETURN_LAUNCH();
}

}  // namespace nnis

// The merge alone, for kernels that write the same partial records.
extern "C" int nnis_attention_merge_bf16(const float* partial, void* out, long long n_rows, int d,
                                         int n_splits, cudaStream_t stream) {
    nnis::attn_merge_kernel<nnis::bf16><<<(unsigned)((n_rows + 3) / 4), 128, 0, stream>>>(
        partial, (nnis::bf16*)out, (size_t)n_rows, d, n_splits);
    NNIS_RETURN_LAUNCH();
}

// Scratch: `partial` needs n_tokens * nq * n_splits * (d + 2) floats when
// n_splits > 1 and may be null otherwise.
NNIS_API int nnis_attention_generic(const void* q, int q_stride, const void* k_cache,
                                    const void* v_cache, const int* token_pos, const int* token_seq,
                                    const int* page_table, int table_cols, void* out, float* partial,
                                    int n_tokens, int nq, int nkv, int d, int page_size, int window,
                                    float scale, int n_splits, int dtype, cudaStream_t stream) {
    if (n_tokens <= 0 || nq <= 0 || nkv <= 0 || nq % nkv || page_size <= 0 || table_cols <= 0 ||
        n_splits <= 0 || window < 0)
        return NNIS_ERR_ARGUMENT;
    if (d <= 0 || d % 2 || d > 256) return NNIS_ERR_UNSUPPORTED;
    if (nq > 65535 || n_splits > 65535) return NNIS_ERR_UNSUPPORTED;
    if (n_splits > 1 && !partial) return NNIS_ERR_ARGUMENT;
    if (dtype == NNIS_DTYPE_F32)
        return nnis::launch_attention<float>(q, q_stride, k_cache, v_cache, token_pos, token_seq,
                                             page_table, table_cols, out, partial, n_tokens, nq, nkv,
                                             d, page_size, window, scale, n_splits, stream);
    if (dtype == NNIS_DTYPE_BF16)
        return nnis::launch_attention<nnis::bf16>(q, q_stride, k_cache, v_cache, token_pos,
                                                  token_seq, page_table, table_cols, out, partial,
                                                  n_tokens, nq, nkv, d, page_size, window, scale,
                                                  n_splits, stream);
    return NNIS_ERR_UNSUPPORTED;
}
