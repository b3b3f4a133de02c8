// Prompt attention over the paged bfloat16 cache on the tensor cores, for head
// sizes 64 and 128: packed query tokens of several sequences, each query seeing
// the keys of its own sequence up to its own position (and within the window, if
// there is one).  The keys and values of the step's own tokens are in the cache
// already, so a sequence may bring a whole prompt or a later chunk of it.
//
// One CTA of four warps owns 64 consecutive query tokens of one sequence and one
// query head, each warp 16 rows of an m16n8k16 tile.  (The kernel is written for
// MT row tiles per warp; two tiles per warp halve the shared-memory reads per
// product but, with 128-query CTAs, left a single 2,048-token prompt with too few
// and too unequal CTAs, and measured slower.)  It walks the sequence's
// pages (64 keys) up to its last query: K and V pages come into swizzled shared
// memory with 16-byte cp.async copies, two pages ahead; scores S = Q K^T and the
// update O += P V are matrix products; the online softmax between them is float32
// in registers (the running maximum and sum per row, exp2 of scaled scores).
// The host lists the tiles (sequence, first query) because sequences have unequal
// lengths.
// NNIS has a batched causal kernel on CUDA cores (crates/nnis-kernels/src/attention.rs:46-150)
// and feeds prompts to its model one token at a time (crates/nnis-model/src/runtime.rs:901-916).
#include <float.h>

#include "mma_helpers.cuh"

namespace nnis {

constexpr int kPrefillRows = 64;   // query rows per CTA
constexpr int kPrefillPage = 64;
constexpr int kPrefillStages = 3;

// MT row tiles of 16 per warp; 128 / (16 MT) warps
template <int D, int MT>
__global__ void __launch_bounds__(kPrefillRows / (16 * MT) * 32)
attn_prefill_mma_kernel(const bf16* __restrict__ q, int q_stride, const bf16* __restrict__ k_cache,
                        const bf16* __restrict__ v_cache, const int* __restrict__ tiles,
                        const int* __restrict__ seq_first_row, const int* __restrict__ seq_start,
                        const int* __restrict__ seq_count, const int* __restrict__ page_table,
                        int table_cols, bf16* __restrict__ out, int nq, int nkv, int window,
                        float scale) {
    constexpr int CH = D / 8, NT = D / 8, KS = D / 16;
    constexpr int kPrefillWarps = kPrefillRows / (16 * MT);
    constexpr int WR = 16 * MT;  // rows per warp
    extern __shared__ __align__(128) unsigned char smem_raw[];
    bf16* q_s = reinterpret_cast<bf16*>(smem_raw);                  // [64, D] swizzled
    bf16* kv_s = q_s + kPrefillRows * D;                            // stages x (K, V) [64, D]

    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, tid = threadIdx.x;
    const int seq = tiles[2 * blockIdx.x], q0 = tiles[2 * blockIdx.x + 1];
    const int hq = blockIdx.y, hk = hq / (nq / nkv);
    const int count = seq_count[seq], start = seq_start[seq];
    const int row_base = seq_first_row[seq] + q0;      // packed row of this tile's first query
    const int rows = min(kPrefillRows, count - q0);    // valid queries in the tile
    const int pos0 = start + q0;                       // position of the first query
    const int hi = pos0 + rows;                        // keys below this position may be seen
    const int lo = window > 0 ? max(0, pos0 - window + 1) : 0;
    const int first_page = lo / kPrefillPage, n_pages = (hi - 1) / kPrefillPage - first_page + 1;
    const int* table = page_table + (size_t)seq * table_cols;
    const size_t tile_elems = (size_t)kPrefillPage * D;

    auto load_page = [&](int it) {
        if (it < n_pages) {
            int page = table[first_page + it];
            const bf16* ksrc = k_cache + (size_t)(page * nkv + hk) * tile_elems;
            const bf16* vsrc = v_cache + (size_t)(page * nkv + hk) * tile_elems;
            bf16* kd = kv_s + (size_t)(it % kPrefillStages) * 2 * tile_elems;
            bf16* vd = kd + tile_elems;
            for (int c = tid; c < kPrefillPage * CH; c += kPrefillWarps * 32) {
                int row = c / CH, chunk = c % CH;
                cp_async16(kd + swz<D>(row, chunk), ksrc + (size_t)c * 8);
                cp_async16(vd + swz<D>(row, chunk), vsrc + (size_t)c * 8);
            }
        }
        cp_async_commit();
    };
    for (int it = 0; it < kPrefillStages - 1; ++it) load_page(it);

    // the tile's queries (rows beyond the sequence are zero)
    for (int c = tid; c < kPrefillRows * CH; c += kPrefillWarps * 32) {
        int row = c / CH, chunk = c % CH;
        uint4 v = make_uint4(0, 0, 0, 0);
        if (row < rows)
            v = *reinterpret_cast<const uint4*>(q + (size_t)(row_base + row) * q_stride +
                                                (size_t)hq * D + chunk * 8);
        *reinterpret_cast<uint4*>(q_s + swz<D>(row, chunk)) = v;
    }
    __syncthreads();
    uint32_t qa[MT][KS][4];
#pragma unroll
    for (int t = 0; t < MT; ++t)
#pragma unroll
        for (int kk = 0; kk < KS; ++kk)
            ldmatrix_x4(qa[t][kk], q_s + swz<D>(warp * WR + t * 16 + (lane & 15), kk * 2 + (lane >> 4)));

    const int r_lo = lane >> 2, c_lo = (lane & 3) * 2;
    // positions of this thread's rows: tile t, rows r_lo and r_lo + 8
    int pos_r[MT][2], lo_r[MT][2];
#pragma unroll
    for (int t = 0; t < MT; ++t)
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            pos_r[t][h] = pos0 + warp * WR + t * 16 + r_lo + h * 8;
            lo_r[t][h] = window > 0 ? pos_r[t][h] - window + 1 : 0;
        }

    float o[MT][NT][4];
    float m_run[MT][2], l_run[MT][2];
#pragma unroll
    for (int t = 0; t < MT; ++t) {
#pragma unroll
        for (int j = 0; j < NT; ++j)
#pragma unroll
            for (int e = 0; e < 4; ++e) o[t][j][e] = 0.f;
        m_run[t][0] = m_run[t][1] = -INFINITY;
        l_run[t][0] = l_run[t][1] = 0.f;
    }
    const float sc = scale * kLog2e;

    for (int it = 0; it < n_pages; ++it) {
        cp_async_wait<kPrefillStages - 2>();
        __syncthreads();
        load_page(it + kPrefillStages - 1);
        const bf16* kt = kv_s + (size_t)(it % kPrefillStages) * 2 * tile_elems;
        const bf16* vt = kt + tile_elems;
        const int t0 = (first_page + it) * kPrefillPage;
        // a warp whose rows all lie before this page has nothing to see in it
        if (t0 > pos0 + warp * WR + WR - 1) continue;

        float s[MT][8][4];
#pragma unroll
        for (int t = 0; t < MT; ++t)
#pragma unroll
            for (int j = 0; j < 8; ++j)
#pragma unroll
                for (int e = 0; e < 4; ++e) s[t][j][e] = 0.f;
#pragma unroll
        for (int kk = 0; kk < KS; kk += 2) {
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                uint32_t b[4];
                ldmatrix_x4(b, kt + swz<D>(j * 8 + (lane & 7), kk * 2 + (lane >> 3)));
#pragma unroll
                for (int t = 0; t < MT; ++t) {
                    mma_bf16(s[t][j], qa[t][kk], b[0], b[1]);
                    mma_bf16(s[t][j], qa[t][kk + 1], b[2], b[3]);
                }
            }
        }
        uint32_t pa[MT][4][4];  // four k-steps of 16 keys
#pragma unroll
        for (int t = 0; t < MT; ++t) {
            float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
            for (int j = 0; j < 8; ++j)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    int key = t0 + j * 8 + c_lo + (e & 1);
                    bool ok = key <= pos_r[t][e >> 1] && key >= lo_r[t][e >> 1];
                    float v = ok ? s[t][j][e] * sc : -INFINITY;
                    s[t][j][e] = v;
                    mx[e >> 1] = fmaxf(mx[e >> 1], v);
                }
            float alpha[2], base[2];
#pragma unroll
            for (int r = 0; r < 2; ++r) {
                mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
                mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
                float mn = fmaxf(m_run[t][r], mx[r]);
                base[r] = mn == -INFINITY ? 0.f : mn;
                alpha[r] = exp2f(m_run[t][r] - base[r]);
                m_run[t][r] = mn;
            }
            float psum[2] = {0.f, 0.f};
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                float p0v = exp2f(s[t][j][0] - base[0]), p1v = exp2f(s[t][j][1] - base[0]);
                float p2v = exp2f(s[t][j][2] - base[1]), p3v = exp2f(s[t][j][3] - base[1]);
                psum[0] += p0v + p1v;
                psum[1] += p2v + p3v;
                pa[t][j >> 1][(j & 1) * 2] = pack_bf16(p0v, p1v);
                pa[t][j >> 1][(j & 1) * 2 + 1] = pack_bf16(p2v, p3v);
            }
#pragma unroll
            for (int r = 0; r < 2; ++r) l_run[t][r] = l_run[t][r] * alpha[r] + psum[r];
#pragma unroll
            for (int jn = 0; jn < NT; ++jn)
#pragma unroll
                for (int e = 0; e < 4; ++e) o[t][jn][e] *= alpha[e >> 1];
        }
#pragma unroll
        for (int ks = 0; ks < 4; ++ks) {
#pragma unroll
            for (int jn = 0; jn < NT; jn += 2) {
                uint32_t b[4];
                ldmatrix_x4_trans(b, vt + swz<D>(ks * 16 + (lane & 15), jn + (lane >> 4)));
#pragma unroll
                for (int t = 0; t < MT; ++t) {
                    mma_bf16(o[t][jn], pa[t][ks], b[0], b[1]);
                    mma_bf16(o[t][jn + 1], pa[t][ks], b[2], b[3]);
                }
            }
        }
    }
    cp_async_wait<0>();
#pragma unroll
    for (int t = 0; t < MT; ++t) {
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            l_run[t][r] += __shfl_xor_sync(0xffffffffu, l_run[t][r], 1);
            l_run[t][r] += __shfl_xor_sync(0xffffffffu, l_run[t][r], 2);
        }
        const float inv_a = l_run[t][0] > 0.f ? 1.0f / l_run[t][0] : 0.f;
        const float inv_b = l_run[t][1] > 0.f ? 1.0f / l_run[t][1] : 0.f;
        const int ra = warp * WR + t * 16 + r_lo, rb = ra + 8;
#pragma unroll
        for (int jn = 0; jn < NT; ++jn) {
            int col = hq * D + jn * 8 + c_lo;
            if (ra < rows)
                *reinterpret_cast<uint32_t*>(out + (size_t)(row_base + ra) * nq * D + col) =
                    pack_bf16(o[t][jn][0] * inv_a, o[t][jn][1] * inv_a);
            if (rb < rows)
                *reinterpret_cast<uint32_t*>(out + (size_t)(row_base + rb) * nq * D + col) =
                    pack_bf16(o[t][jn][2] * inv_b, o[t][jn][3] * inv_b);
        }
    }
}

template <int D, int MT>
static int launch_prefill(dim3 grid, cudaStream_t stream, const bf16* q, int q_stride, const bf16* k,
                          const bf16* v, const int* tiles, const int* first_row, const int* start,
                          const int* count, const int* table, int cols, bf16* out, int nq, int nkv,
                          int window, float scale) {
    size_t smem = ((size_t)kPrefillRows * D + (size_t)kPrefillStages * 2 * kPrefillPage * D) * sizeof(bf16);
    auto kernel = attn_prefill_mma_kernel<D, MT>;
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             (int)smem);
        if (e != cudaSuccess) return (int)e;
    }
    kernel<<<grid, kPrefillRows / (16 * MT) * 32, smem, stream>>>(q, q_stride, k, v, tiles, first_row, start,
                                                       count, table, cols, out, nq, nkv, window, scale);
    NNIS_RETURN_LAUNCH();
}

}  // namespace nnis

// `tiles`: int32 [n_tiles, 2] = (sequence of the batch, first query of the tile
// within this step's tokens of that sequence), 64 queries per tile.  Per
// sequence: `seq_first_row` the packed row of its first token of this step,
// `seq_start` that token's position, `seq_count` its number of tokens.  Takes
// head sizes 64 and 128 with 64-key pages; else NNIS_ERR_UNSUPPORTED.
NNIS_API int nnis_attention_prefill_mma(const void* q, int q_stride, const void* k_cache,
                                        const void* v_cache, const int* tiles, int n_tiles,
                                        const int* seq_first_row, const int* seq_start,
                                        const int* seq_count, const int* page_table, int table_cols,
                                        void* out, int nq, int nkv, int d, int page_size, int window,
                                        float scale, cudaStream_t stream) {
    using namespace nnis;
    if (n_tiles <= 0 || nq <= 0 || nkv <= 0 || nq % nkv || table_cols <= 0 || window < 0 || !tiles)
        return NNIS_ERR_ARGUMENT;
    if ((d != 64 && d != 128) || page_size != kPrefillPage) return NNIS_ERR_UNSUPPORTED;
    if (nq > 65535) return NNIS_ERR_UNSUPPORTED;
    if (((uintptr_t)q | (uintptr_t)k_cache | (uintptr_t)v_cache | (uintptr_t)out) % 16 ||
        (q_stride % 8))
        return NNIS_ERR_ALIGNMENT;
    dim3 grid(n_tiles, nq);
    if (d == 64)
        return launch_prefill<64, 1>(grid, stream, (const bf16*)q, q_stride, (const bf16*)k_cache,
                                  (const bf16*)v_cache, tiles, seq_first_row, seq_start, seq_count,
                                  page_table, table_cols, (bf16*)out, nq, nkv, window, scale);
    return launch_prefill<128, 1>(grid, stream, (const bf16*)q, q_stride, (const bf16*)k_cache,
                               (const bf16*)v_cache, tiles, seq_first_row, seq_start, seq_count,
                               page_table, table_cols, (bf16*)out, nq, nkv, window, scale);
}
