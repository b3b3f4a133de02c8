// Decode attention over the paged bfloat16 cache on the tensor cores, for head
// sizes 64 and 128: one query token per sequence against its whole context.
//
// The query heads that share a kv head (up to 16) form the 16 rows of an
// m16n8k16 tile, so K and V are read once for the whole group and the scores and
// the weighted sum of values are matrix products; the softmax between them stays
// in float32 registers.  One CTA of four warps owns (kv head, group of query
// heads, sequence, slice of the key range).  Pages of K and V (64 keys) come
// into shared memory with 16-byte cp.async copies, several pages ahead, into
// rows whose 16-byte chunks are XOR-swizzled so that ldmatrix meets no bank
// conflict; each warp takes 16 keys of every page and keeps its own running
// (max, sum, output); warps are merged through shared memory at the end.  With
// several slices the partial results go to scratch, and the slice that arrives
// last (a ticket per group) merges them, in a fixed order, into the output.
//
// The step is bound by the bytes of K and V; the tensor cores are here to keep
// the instruction count per byte low, not for their throughput.
// NNIS: crates/nnis-model/src/kernels.rs:66-125 (one thread per query head).
#include <float.h>

#include "async_copy.cuh"
#include "common.cuh"
#include "mma_helpers.cuh"

namespace nnis {

constexpr int kMmaWarps = 4;
constexpr int kPage = 64;
template <int D>
__global__ void __launch_bounds__(kMmaWarps * 32)
attn_decode_mma_kernel(const bf16* __restrict__ q, int q_stride, const bf16* __restrict__ k_cache,
                       const bf16* __restrict__ v_cache, const int* __restrict__ token_pos,
                       const int* __restrict__ token_seq, const int* __restrict__ page_table,
                       int table_cols, bf16* __restrict__ out, float* __restrict__ partial,
                       unsigned* __restrict__ tickets, int nq, int nkv, int window, float scale,
                       int n_splits, int head_tiles, int stages, unsigned long long* trace) {
    trace_mark(trace, 0);
    constexpr int CH = D / 8;    // 16-byte chunks per row
    constexpr int NT = D / 8;    // n-tiles of the output
    constexpr int KS = D / 16;   // k-steps of the score product
    extern __shared__ __align__(128) unsigned char smem_raw[];
    bf16* q_s = reinterpret_cast<bf16*>(smem_raw);           // [16, D] swizzled
    bf16* tiles = q_s + 16 * D;                              // stages x (K [64, D], V [64, D])
    __shared__ float sm_ml[kMmaWarps][16][2];
    __shared__ bool is_last;

    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, tid = threadIdx.x;
    const int hk = blockIdx.x / head_tiles, tile = blockIdx.x % head_tiles;
    const int G = nq / nkv;
    const int g0 = tile * 16;
    const int gcount = min(16, G - g0);
    const int n = blockIdx.y, split = blockIdx.z;

    // Slices are fixed ranges of the page table (not of this sequence's length), so
    // the page ids of a slice can be asked for together with the position instead
    // of after it.
    // Under programmatic dependent launch this kernel may start while the kernel
    // before it (the one that writes this step's query, key and value) still runs.
    // Every kernel of the step releases its dependents only after its own wait, so
    // all kernels before that one are complete: positions, page tables and every
    // cache page except the one that holds this step's token may be read at once.
    const int per = (table_cols + n_splits - 1) / n_splits;
    const int p0 = split * per;
    const int* table = page_table + (size_t)token_seq[n] * table_cols;
    const int pos = token_pos[n];
    int first_ids[3];
#pragma unroll
    for (int i = 0; i < 3; ++i) first_ids[i] = (i < per && p0 + i < table_cols) ? table[p0 + i] : 0;
    const int r_lo = lane >> 2, c_lo = (lane & 3) * 2;  // this thread's rows r_lo, r_lo + 8

    float o[NT][4];
#pragma unroll
    for (int j = 0; j < NT; ++j)
#pragma unroll
        for (int e = 0; e < 4; ++e) o[j][e] = 0.f;
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};

    if (pos >= 0) {
        const int lo = window > 0 ? max(0, pos - window + 1) : 0;
        const int hi = pos + 1;
        const int first_page = lo / kPage, last_page = (hi - 1) / kPage;
        // this slice's pages that the query can see: [begin, begin + count)
        const int begin = max(p0, first_page);
        const int count = max(0, min(last_page + 1, p0 + per) - begin);
        const size_t tile_elems = (size_t)kPage * D;

        auto load_page = [&](int it) {
            if (it < count) {
                int idx = begin + it - p0;  // place within the slice
                int page = idx < 3 ? (idx == 0 ? first_ids[0] : idx == 1 ? first_ids[1] : first_ids[2])
                                   : table[begin + it];
                const bf16* ksrc = k_cache + (size_t)(page * nkv + hk) * tile_elems;
                const bf16* vsrc = v_cache + (size_t)(page * nkv + hk) * tile_elems;
                bf16* kd = tiles + (size_t)(it % stages) * 2 * tile_elems;
                bf16* vd = kd + tile_elems;
                for (int c = tid; c < kPage * CH; c += kMmaWarps * 32) {
                    int row = c / CH, chunk = c % CH;
                    cp_async16(kd + swz<D>(row, chunk), ksrc + (size_t)c * 8);
                    cp_async16(vd + swz<D>(row, chunk), vsrc + (size_t)c * 8);
                }
            }
            cp_async_commit();
        };
        // the page of this step's token is the last one of the sequence: it waits
        const int hot = last_page - begin;
        int issued = 0;
        for (; issued < stages - 1 && issued != hot; ++issued) load_page(issued);
        pdl_wait();
        pdl_launch_dependents();
        trace_mark(trace, 2);
        trace_mark(trace, 3);
        for (; issued < stages - 1; ++issued) load_page(issued);

        // the group's query rows, zero beyond the group
        for (int c = tid; c < 16 * CH; c += kMmaWarps * 32) {
            int row = c / CH, chunk = c % CH;
            uint4 v = make_uint4(0, 0, 0, 0);
            if (row < gcount)
                v = *reinterpret_cast<const uint4*>(q + (size_t)n * q_stride +
                                                    (size_t)(hk * G + g0 + row) * D + chunk * 8);
            *reinterpret_cast<uint4*>(q_s + swz<D>(row, chunk)) = v;
        }
        __syncthreads();
        uint32_t qa[KS][4];
#pragma unroll
        for (int kk = 0; kk < KS; ++kk)
            ldmatrix_x4(qa[kk], q_s + swz<D>(lane & 15, kk * 2 + (lane >> 4)));

        const float sc = scale * kLog2e;
        for (int it = 0; it < count; ++it) {
            if (stages == 2) cp_async_wait<0>();
            else if (stages == 3) cp_async_wait<1>();
            else cp_async_wait<2>();
            __syncthreads();  // page `it` has landed for everyone; the stage of page it-1 is free
            load_page(it + stages - 1);
            const bf16* kt = tiles + (size_t)(it % stages) * 2 * tile_elems;
            const bf16* vt = kt + tile_elems;
            const int key0 = warp * 16;  // this warp's 16 keys of the page
            const int t0 = (begin + it) * kPage + key0;

            // scores: S[16 heads, 16 keys] = Q . K^T
            float s[2][4];
#pragma unroll
            for (int j = 0; j < 2; ++j)
#pragma unroll
                for (int e = 0; e < 4; ++e) s[j][e] = 0.f;
            // all fragments of K first, then the products: none waits for the load just ahead of it
            uint32_t kb[KS / 2][2][4];
#pragma unroll
            for (int kk = 0; kk < KS; kk += 2)
#pragma unroll
                for (int j = 0; j < 2; ++j)
                    // four 8x8 tiles: keys j*8.., dims kk*16 .. kk*16+31
                    ldmatrix_x4(kb[kk / 2][j], kt + swz<D>(key0 + j * 8 + (lane & 7), kk * 2 + (lane >> 3)));
#pragma unroll
            for (int kk = 0; kk < KS; kk += 2) {
#pragma unroll
                for (int j = 0; j < 2; ++j) {
                    mma_bf16(s[j], qa[kk], kb[kk / 2][j][0], kb[kk / 2][j][1]);
                    mma_bf16(s[j], qa[kk + 1], kb[kk / 2][j][2], kb[kk / 2][j][3]);
                }
            }
            // mask, scale (in log2 units) and this slice's row maxima
            float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
            for (int j = 0; j < 2; ++j)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    int t = t0 + j * 8 + c_lo + (e & 1);
                    float v = (t >= lo && t < hi) ? s[j][e] * sc : -INFINITY;
                    s[j][e] = v;
                    mx[e >> 1] = fmaxf(mx[e >> 1], v);
                }
#pragma unroll
            for (int r = 0; r < 2; ++r) {
                mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
                mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
            }
            float alpha[2], base[2];
#pragma unroll
            for (int r = 0; r < 2; ++r) {
                float mn = fmaxf(m_run[r], mx[r]);
                base[r] = mn == -INFINITY ? 0.f : mn;  // nothing seen yet: avoid inf - inf
                alpha[r] = exp2f(m_run[r] - base[r]);
                m_run[r] = mn;
            }
            uint32_t pa[4];
            float psum[2] = {0.f, 0.f};
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                float p0v = exp2f(s[j][0] - base[0]), p1v = exp2f(s[j][1] - base[0]);
                float p2v = exp2f(s[j][2] - base[1]), p3v = exp2f(s[j][3] - base[1]);
                psum[0] += p0v + p1v;
                psum[1] += p2v + p3v;
                pa[j * 2] = pack_bf16(p0v, p1v);
                pa[j * 2 + 1] = pack_bf16(p2v, p3v);
            }
#pragma unroll
            for (int r = 0; r < 2; ++r) l_run[r] = l_run[r] * alpha[r] + psum[r];
            // output: O = O * alpha + P . V
            // the fragments of V four tiles ahead of their products
            constexpr int kAhead = 4;  // pairs of n-tiles in flight
#pragma unroll
            for (int j0 = 0; j0 < NT; j0 += 2 * kAhead) {
                uint32_t vb[kAhead][4];
#pragma unroll
                for (int a = 0; a < kAhead; ++a)
                    // keys 0-7 / 8-15 of this warp's slice, dims jn*8 .. jn*8+15
                    if (j0 + 2 * a < NT)
                        ldmatrix_x4_trans(vb[a], vt + swz<D>(key0 + (lane & 15), j0 + 2 * a + (lane >> 4)));
#pragma unroll
                for (int a = 0; a < kAhead; ++a) {
                    const int jn = j0 + 2 * a;
                    if (jn < NT) {
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            o[jn][e] *= alpha[e >> 1];
                            o[jn + 1][e] *= alpha[e >> 1];
                        }
                        mma_bf16(o[jn], pa, vb[a][0], vb[a][1]);
                        mma_bf16(o[jn + 1], pa, vb[a][2], vb[a][3]);
                    }
                }
            }
        }
        cp_async_wait<0>();
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 1);
            l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 2);
        }
    }
    if (pos < 0) {
        pdl_wait();
        pdl_launch_dependents();
    }
    __syncthreads();  // everyone is done with the tiles: reuse them for the merge
    trace_mark(trace, 4);
    trace_mark(trace, 5);

    // ---- merge the four warps: (m, l) through sm_ml, outputs through the tiles ----
    float* o_s = reinterpret_cast<float*>(smem_raw);  // [warps, 16, D] float32
    if ((lane & 3) == 0) {
        sm_ml[warp][r_lo][0] = m_run[0];
        sm_ml[warp][r_lo][1] = l_run[0];
        sm_ml[warp][r_lo + 8][0] = m_run[1];
        sm_ml[warp][r_lo + 8][1] = l_run[1];
    }
#pragma unroll
    for (int j = 0; j < NT; ++j) {
        float* base0 = o_s + ((size_t)warp * 16 + r_lo) * D + j * 8 + c_lo;
        base0[0] = o[j][0];
        base0[1] = o[j][1];
        base0[8 * D] = o[j][2];
        base0[8 * D + 1] = o[j][3];
    }
    __syncthreads();
    // thread -> (row, 8 dims); 16 rows x D/8 chunks = 2 D items over 128 threads
    for (int item = tid; item < 16 * CH; item += kMmaWarps * 32) {
        int row = item / CH, chunk = item % CH;
        if (row >= gcount) continue;
        float mm = -INFINITY;
#pragma unroll
        for (int w = 0; w < kMmaWarps; ++w) mm = fmaxf(mm, sm_ml[w][row][0]);
        float ll = 0.f, acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        if (mm != -INFINITY) {
#pragma unroll
            for (int w = 0; w < kMmaWarps; ++w) {
                float f = exp2f(sm_ml[w][row][0] - mm);
                ll += sm_ml[w][row][1] * f;
                const float* src = o_s + ((size_t)w * 16 + row) * D + chunk * 8;
#pragma unroll
                for (int e = 0; e < 8; ++e) acc[e] = fmaf(src[e], f, acc[e]);
            }
        }
        int hq = hk * G + g0 + row;
        if (n_splits == 1) {
            float inv = ll > 0.f ? 1.0f / ll : 0.f;
            bf16* dst = out + ((size_t)n * nq + hq) * D + chunk * 8;
            store4(dst, make_float4(acc[0] * inv, acc[1] * inv, acc[2] * inv, acc[3] * inv));
            store4(dst + 4, make_float4(acc[4] * inv, acc[5] * inv, acc[6] * inv, acc[7] * inv));
        } else {
            float* rec = partial + (((size_t)n * nq + hq) * n_splits + split) * (size_t)(D + 2);
            if (chunk == 0) {
                rec[0] = mm;  // log2 units
                rec[1] = ll;
            }
#pragma unroll
            for (int e = 0; e < 8; ++e) rec[2 + chunk * 8 + e] = acc[e];
        }
    }
    if (n_splits == 1) {
        trace_mark(trace, 1);
        return;
    }

    // ---- the slice that arrives last merges all slices of its group ----------------
    // One thread takes the ticket: its fence, after the barrier, also covers what the
    // other threads of the CTA wrote before the barrier.
    __syncthreads();
    unsigned* ticket = tickets + ((size_t)n * nkv + hk) * head_tiles + tile;
    if (tid == 0) {
        __threadfence();
        is_last = atomicAdd(ticket, 1u) == (unsigned)n_splits - 1u;
    }
    __syncthreads();
    trace_mark(trace, 6);
    trace_mark(trace, 7);
    if (!is_last) {
        trace_mark(trace, 1);
        return;
    }
    __threadfence();
    // One trip to L2: a thread owns (row, 8 dims, one of four interleaved groups of
    // slices) and asks for the maxima, sums and outputs of its slices all at once;
    // it folds them against the group's own maximum, and the four groups of a row
    // meet in shared memory, added in the order of the groups.
    float* g_ml = reinterpret_cast<float*>(smem_raw);           // [4, 16, 2] group maximum and sum
    float* g_o = g_ml + 4 * 16 * 2;                             // [4, 16, D] group outputs
    constexpr int kRound = 4;  // slices of a group asked for at once (all of them up to 16 slices)
    for (int item = tid; item < gcount * CH * 4; item += kMmaWarps * 32) {
        int grp4 = item & 3, rc = item >> 2;
        int row = rc / CH, chunk = rc % CH;
        const float* rec = partial + ((size_t)n * nq + hk * G + g0 + row) * n_splits * (size_t)(D + 2);
        float mm = -INFINITY, ll = 0.f;
        float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        for (int first = grp4; first < n_splits; first += 4 * kRound) {
            float mv[kRound], lv[kRound];
            float2 ov[kRound][4];
#pragma unroll
            for (int i = 0; i < kRound; ++i) {
                int sp = first + 4 * i;
                mv[i] = -INFINITY;
                lv[i] = 0.f;
                if (sp < n_splits) {
                    const float* r = rec + (size_t)sp * (D + 2);
                    mv[i] = __ldcg(r);
                    lv[i] = __ldcg(r + 1);
                    const float2* o2 = reinterpret_cast<const float2*>(r + 2 + chunk * 8);
#pragma unroll
                    for (int e = 0; e < 4; ++e) ov[i][e] = __ldcg(o2 + e);
                }
            }
            float m_new = mm;
#pragma unroll
            for (int i = 0; i < kRound; ++i)
                if (lv[i] > 0.f) m_new = fmaxf(m_new, mv[i]);
            if (m_new == -INFINITY) continue;
            const float keep = mm == -INFINITY ? 0.f : exp2f(mm - m_new);
            ll *= keep;
#pragma unroll
            for (int e = 0; e < 8; ++e) acc[e] *= keep;
            mm = m_new;
#pragma unroll
            for (int i = 0; i < kRound; ++i) {
                if (lv[i] > 0.f) {
                    float f = exp2f(mv[i] - mm);
                    ll = fmaf(lv[i], f, ll);
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        acc[2 * e] = fmaf(ov[i][e].x, f, acc[2 * e]);
                        acc[2 * e + 1] = fmaf(ov[i][e].y, f, acc[2 * e + 1]);
                    }
                }
            }
        }
        if (chunk == 0) {
            g_ml[(grp4 * 16 + row) * 2] = mm;
            g_ml[(grp4 * 16 + row) * 2 + 1] = ll;
        }
        float* dst = g_o + ((size_t)grp4 * 16 + row) * D + chunk * 8;
#pragma unroll
        for (int e = 0; e < 8; ++e) dst[e] = acc[e];
    }
    __syncthreads();
    for (int item = tid; item < gcount * CH; item += kMmaWarps * 32) {
        int row = item / CH, chunk = item % CH;
        int hq = hk * G + g0 + row;
        float mm = -INFINITY;
#pragma unroll
        for (int g4 = 0; g4 < 4; ++g4) mm = fmaxf(mm, g_ml[(g4 * 16 + row) * 2]);
        float f[4], ll = 0.f;
#pragma unroll
        for (int g4 = 0; g4 < 4; ++g4) {
            float gm = g_ml[(g4 * 16 + row) * 2];
            f[g4] = gm == -INFINITY ? 0.f : exp2f(gm - mm);
            ll = fmaf(g_ml[(g4 * 16 + row) * 2 + 1], f[g4], ll);
        }
        float inv = ll > 0.f ? 1.0f / ll : 0.f;
        float acc[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            const float* src = g_o + (size_t)row * D + chunk * 8 + e;
            acc[e] = ((src[0] * f[0] + src[16 * D] * f[1]) + src[32 * D] * f[2]) + src[48 * D] * f[3];
        }
        bf16* dst = out + ((size_t)n * nq + hq) * D + chunk * 8;
        store4(dst, make_float4(acc[0] * inv, acc[1] * inv, acc[2] * inv, acc[3] * inv));
        store4(dst + 4, make_float4(acc[4] * inv, acc[5] * inv, acc[6] * inv, acc[7] * inv));
    }
    if (tid == 0) *ticket = 0u;
    trace_mark(trace, 1);
}

template <int D>
constexpr int mma_stages() { return D <= 64 ? 4 : 3; }
// `stages`: pages of K and V in flight per CTA, 2 to the default (0: the default).
// One stage less lets another CTA live on the SM (four instead of three at head
// size 64), which pays when the step's CTAs then fill one wave.
template <int D>
static int mma_stages_or_default(int stages) {
    return stages >= 2 && stages <= mma_stages<D>() ? stages : mma_stages<D>();
}
template <int D>
static size_t mma_smem_bytes(int stages) {
    size_t stage_bytes = 2 * (size_t)kPage * D * sizeof(bf16);
    size_t smem = 16 * D * sizeof(bf16) + stages * stage_bytes;
    size_t merge_bytes = ((size_t)kMmaWarps * 16 * D + 4 * 16 * 2) * sizeof(float);
    return smem < merge_bytes ? merge_bytes : smem;
}

template <int D>
static int resident_ctas_per_sm(int stages) {
    auto kernel = attn_decode_mma_kernel<D>;
    const size_t smem = mma_smem_bytes<D>(mma_stages_or_default<D>(stages));
    if (smem > 48 * 1024 &&
        cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) !=
            cudaSuccess)
        return 0;
    int blocks = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&blocks, kernel, kMmaWarps * 32, smem) !=
        cudaSuccess)
        return 0;
    return blocks;
}

template <int D>
static int launch_mma(dim3 grid, bool pdl, cudaStream_t stream, const bf16* q, int q_stride,
                      const bf16* k, const bf16* v, const int* pos, const int* seq, const int* table,
                      int cols, bf16* out, float* partial, unsigned* tickets, int nq, int nkv,
                      int window, float scale, int n_splits, int head_tiles, int want_stages) {
    const int stages = mma_stages_or_default<D>(want_stages);
    const size_t smem = mma_smem_bytes<D>(stages);
    auto kernel = attn_decode_mma_kernel<D>;
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             (int)smem);
        if (e != cudaSuccess) return (int)e;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(kMmaWarps * 32);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 1 : 0;
    cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, q, q_stride, k, v, pos, seq, table, cols, out,
                                       partial, tickets, nq, nkv, window, scale, n_splits, head_tiles,
                                       stages, trace_slot("attention decode"));
    return e == cudaSuccess ? NNIS_OK : (int)e;
}

}  // namespace nnis

// How many CTAs of the kernel for head size `d` one SM holds at a time (0: head
// size not taken, or the query failed).  The host cuts the key range so that all
// CTAs of a step are resident together: a second, partly filled wave costs more
// than shorter slices gain.
NNIS_API int nnis_attention_decode_mma_ctas_per_sm(int d, int stages) {
    if (d == 64) return nnis::resident_ctas_per_sm<64>(stages);
    if (d == 128) return nnis::resident_ctas_per_sm<128>(stages);
    return 0;
}

// The default number of stages for head size `d` (0: head size not taken).
NNIS_API int nnis_attention_decode_mma_stages(int d) {
    return d == 64 ? nnis::mma_stages<64>() : d == 128 ? nnis::mma_stages<128>() : 0;
}

// Takes head sizes 64 and 128 with 64-key pages; anything else is refused with
// NNIS_ERR_UNSUPPORTED and goes to the general decode kernel.  Scratch: with
// n_splits > 1, `partial` (n_tokens * nq * n_splits * (d + 2) floats) and
// `tickets` (n_tokens * nkv * ceil(group / 16) counters, zero before the first
// launch; the kernel leaves them zero).
NNIS_API int nnis_attention_decode_mma_staged(const void* q, int q_stride, const void* k_cache,
                                              const void* v_cache, const int* token_pos,
                                              const int* token_seq, const int* page_table,
                                              int table_cols, void* out, float* partial,
                                              unsigned* tickets, int n_tokens, int nq, int nkv, int d,
                                              int page_size, int window, float scale, int n_splits,
                                              int stages, int pdl, cudaStream_t stream) {
    using namespace nnis;
    if (n_tokens <= 0 || nq <= 0 || nkv <= 0 || nq % nkv || table_cols <= 0 || n_splits <= 0 ||
        window < 0)
        return NNIS_ERR_ARGUMENT;
    if ((d != 64 && d != 128) || page_size != kPage) return NNIS_ERR_UNSUPPORTED;
    if (n_tokens > 65535 || n_splits > 64) return NNIS_ERR_UNSUPPORTED;
    if (n_splits > 1 && (!partial || !tickets)) return NNIS_ERR_ARGUMENT;
    if (((uintptr_t)q | (uintptr_t)k_cache | (uintptr_t)v_cache | (uintptr_t)out) % 16 ||
        (q_stride % 8))
        return NNIS_ERR_ALIGNMENT;
    int G = nq / nkv;
    int head_tiles = (G + 15) / 16;
    dim3 grid(nkv * head_tiles, n_tokens, n_splits);
    if (d == 64)
        return launch_mma<64>(grid, pdl != 0, stream, (const bf16*)q, q_stride, (const bf16*)k_cache,
                              (const bf16*)v_cache, token_pos, token_seq, page_table, table_cols,
                              (bf16*)out, partial, tickets, nq, nkv, window, scale, n_splits,
                              head_tiles, stages);
    return launch_mma<128>(grid, pdl != 0, stream, (const bf16*)q, q_stride, (const bf16*)k_cache,
                           (const bf16*)v_cache, token_pos, token_seq, page_table, table_cols,
                           (bf16*)out, partial, tickets, nq, nkv, window, scale, n_splits, head_tiles,
                           stages);
}

// The same with the default number of stages.
NNIS_API int nnis_attention_decode_mma(const void* q, int q_stride, const void* k_cache,
                                       const void* v_cache, const int* token_pos,
                                       const int* token_seq, const int* page_table, int table_cols,
                                       void* out, float* partial, unsigned* tickets, int n_tokens,
                                       int nq, int nkv, int d, int page_size, int window, float scale,
                                       int n_splits, int pdl, cudaStream_t stream) {
    return nnis_attention_decode_mma_staged(q, q_stride, k_cache, v_cache, token_pos, token_seq,
                                            page_table, table_cols, out, partial, tickets, n_tokens,
                                            nq, nkv, d, page_size, window, scale, n_splits, 0, pdl,
                                            stream);
}
