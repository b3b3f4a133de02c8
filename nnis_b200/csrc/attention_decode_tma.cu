// Decode attention for few sequences, head sizes 64 and 128, with every page of a
// slice in shared memory at once, brought there by TMA.
//
// As in attention_decode_mma.cu the query heads that share a kv head (up to 16) are
// the rows of m16n8k16 tiles, a CTA owns (kv head, group of query heads, sequence,
// slice of the key range), the softmax state is float32, and with several slices the
// partial records meet in scratch where the slice that arrives last at a ticket merges
// them in a fixed order.  That kernel streams slices of any length through a ring of
// stages filled by 16-byte cp.async copies; what bounds a decode step of a small model
// at batch 1 to 8 is the chain of its kernels, in which the attention kernel is the
// longest link, and three things make this kernel's link shorter:
//
//  * Every page of a slice (at most kMaxPages of 64 keys) has a place of its own in
//    shared memory and comes as two tile loads of the TMA unit (K and V, 128-byte
//    swizzled so that ldmatrix meets no bank conflict), issued by one thread before
//    the wait of programmatic dependent launch.  Nothing of the copy engine's work holds
//    a thread (16-byte copies cost some 150 instructions per warp and page for addresses
//    alone and stall their threads once a few thousand are in flight per SM), and the
//    kernel that computes q may let this one start together with it.
//  * The newest page is asked for with the others: all of it but the row of this step's
//    token is as old as they are, and that one row is fetched again after the wait,
//    beside the query.  After the wait nothing else is still to come.
//  * A warp takes whole pages (64 keys at a time): the four warps of a CTA work on four
//    pages side by side without a barrier between pages, with one rescaling of the
//    running output per page and 32 independent score products in flight.
//
// Measured on a B200 against attention_decode_mma.cu in the decode step of the
// SmolLM2-135M shape at context 4,096: batch 1 +3.4 % tokens a second, batch 8 +2 to 3 %.
// Two further forms were built and measured and are not here.  Slices as the CTAs of a
// thread-block cluster, merged through distributed shared memory: a cluster launch does
// not start early under programmatic dependent launch, at most 21 clusters of 16 such
// CTAs are resident on a B200, and reading sixteen records over the cluster's network
// took as long as the ticket and the trip through L2.  A ring of stages with a fifth
// warp issuing the loads, for slices of any length: 40 % fewer instructions than the
// cp.async kernel and the same 5.1 TB/s at batch 64 (both wait for DRAM there), 2 % on
// the step, but 7 % slower at batch 1.
//
// P is rounded to bfloat16 before P.V as in the other tensor-core attention kernels.
// NNIS: crates/nnis-model/src/kernels.rs:66-125 (one thread per query head, serial keys);
// its split of the key range, crates/nnis-model/src/cached_attention_candidate.rs:16-86.
#include <float.h>
#include <limits.h>

#include "mma_helpers.cuh"
#include "tcgen05_helpers.cuh"

namespace nnis {

constexpr int kClWarps = 4;
constexpr int kClThreads = kClWarps * 32;
constexpr int kClPage = 64;
constexpr int kMaxPages = 8;       // pages of one slice, all in shared memory at once
constexpr int kMaxSlices = 128;

// element offset of 16-byte chunk `chunk` of row `row` in a tile of 64 rows that TMA
// wrote as D / 64 boxes of 64 x 64 elements, each with the 128-byte swizzle
template <int D>
__device__ __forceinline__ int tile_off(int row, int chunk) {
    return (chunk >> 3) * (kClPage * 64) + row * 64 + (((chunk & 7) ^ (row & 7)) << 3);
}

// asks `bytes` (a multiple of 16) at a 16-byte aligned address into L2; nothing waits for it
__device__ __forceinline__ void l2_prefetch(const void* p, uint32_t bytes) {
    asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(p), "r"(bytes) : "memory");
}

// counts an arrival; orders this CTA's earlier writes before it and its later reads after it
__device__ __forceinline__ unsigned ticket_take(unsigned* ticket) {
    unsigned old;
    asm volatile("atom.add.acq_rel.gpu.global.u32 %0, [%1], 1;" : "=r"(old) : "l"(ticket) : "memory");
    return old;
}

// Three CTAs of 167 registers fill an SM's register file; a build held to 96 registers
// (so that three CTAs and a projection's fit together) spilled a few values inside its
// loops and was slower wherever it was tried, with two and with three CTAs to an SM.
template <int D>
__global__ void __launch_bounds__(kClThreads, 3)
attn_decode_tma_kernel(const __grid_constant__ CUtensorMap map_k,
                       const __grid_constant__ CUtensorMap map_v, const bf16* k_cache,
                       const bf16* v_cache, const bf16* __restrict__ q, int q_stride,
                       const int* __restrict__ token_pos, const int* __restrict__ token_seq,
                       const int* __restrict__ page_table, int table_cols, bf16* __restrict__ out,
                       float* __restrict__ partial, unsigned* __restrict__ tickets, int nq, int nkv,
                       int window, float scale, int n_splits, int head_tiles, int per, int* status,
                       long long ahead, unsigned long long* trace) {
    trace_mark(trace, 0);
    constexpr int CH = D / 8;    // 16-byte chunks per row
    constexpr int NT = D / 8;    // n-tiles of the output
    constexpr int KS = D / 16;   // k-steps of the score product
    constexpr int HALVES = D / 64;
    constexpr int TILE = kClPage * D;  // elements of one page of K (or V) of one kv head
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    bf16* q_s = reinterpret_cast<bf16*>(smem_raw);           // [16, D] swizzled (2 or 4 KB)
    bf16* tiles = q_s + 16 * D;                              // per x (K [64, D], V [64, D]), 1 KB aligned
    __shared__ uint64_t bars[kMaxPages];                     // one per page, used once
    __shared__ float sm_ml[kClWarps][16][2];
    __shared__ int ids[kMaxPages];
    __shared__ bool is_last;

    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, tid = threadIdx.x;
    const int hk = blockIdx.x / head_tiles, tile = blockIdx.x % head_tiles;
    const int G = nq / nkv;
    const int g0 = tile * 16;
    const int gcount = min(16, G - g0);
    const int n = blockIdx.y, split = blockIdx.z;

    // Positions, page tables and every cache row except the one of this step's token
    // were complete before the step began (or before the kernel that precedes this
    // one's predecessor ended): they are read before the wait.
    const int p0 = split * per;
    const int* table = page_table + (size_t)token_seq[n] * table_cols;
    const int pos = token_pos[n];
    if (tid == 0) {
        prefetch_tensormap(&map_k);
        prefetch_tensormap(&map_v);
        for (int i = 0; i < per; ++i) mbar_init(bars + i, 1);
        mbar_fence_init();
    }
    if (tid < per) ids[tid] = p0 + tid < table_cols ? table[p0 + tid] : 0;
    __syncthreads();

    const int r_lo = lane >> 2, c_lo = (lane & 3) * 2;  // this thread's rows r_lo, r_lo + 8
    float o[NT][4];
#pragma unroll
    for (int j = 0; j < NT; ++j)
#pragma unroll
        for (int e = 0; e < 4; ++e) o[j][e] = 0.f;
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
    bool failed = false;

    int count = 0, begin = p0, lo = 0, hi = 0, hot = -1;
    if (pos >= 0) {
        lo = window > 0 ? max(0, pos - window + 1) : 0;
        hi = pos + 1;
        const int first_page = lo / kClPage, last_page = (hi - 1) / kClPage;
        // this slice's pages that the query can see: [begin, begin + count)
        begin = max(p0, first_page);
        count = max(0, min(last_page + 1, p0 + per) - begin);
        hot = last_page - begin;  // the page of this step's token, if it is in this slice
    }
    // The newest page is asked for with the others: all of it but the row of this step's
    // token is as old as they are, and that one row is fetched again after the wait.
    if (tid == 0) {
        for (int it = 0; it < count; ++it) {
            bf16* kd = tiles + (size_t)it * 2 * TILE;
            const int row0 = (ids[begin - p0 + it] * nkv + hk) * kClPage;
            mbar_expect_tx(bars + it, 2u * TILE * (uint32_t)sizeof(bf16));
#pragma unroll
            for (int h = 0; h < HALVES; ++h) {
                tma_load_2d(kd + h * kClPage * 64, &map_k, h * 64, row0, bars + it);
                tma_load_2d(kd + TILE + h * kClPage * 64, &map_v, h * 64, row0, bars + it);
            }
        }
    }
    pdl_wait();
    pdl_launch_dependents();
    trace_mark(trace, 2);
    trace_mark(trace, 3);

    if (count > 0) {
        // the group's query rows, zero beyond the group
        for (int c = tid; c < 16 * CH; c += kClThreads) {
            int row = c / CH, chunk = c % CH;
            uint4 v = make_uint4(0, 0, 0, 0);
            if (row < gcount)
                v = *reinterpret_cast<const uint4*>(q + (size_t)n * q_stride +
                                                    (size_t)(hk * G + g0 + row) * D + chunk * 8);
            *reinterpret_cast<uint4*>(q_s + swz<D>(row, chunk)) = v;
        }
        // the key and the value that the kernel before this one has just stored: over
        // what the tile load brought for that row (once that load has landed)
        if (hot >= 0 && hot < count && tid < 2 * CH) {
            const int chunk = tid % CH, is_v = tid / CH, in_page = pos % kClPage;
            const bf16* cache = is_v ? v_cache : k_cache;
            const size_t row = (size_t)(ids[begin - p0 + hot] * nkv + hk) * kClPage + in_page;
            const uint4 v = __ldcg(reinterpret_cast<const uint4*>(cache + row * D + chunk * 8));
            if (!mbar_wait(bars + hot, 0)) failed = true;
            bf16* tile_base = tiles + (size_t)hot * 2 * TILE + (is_v ? TILE : 0);
            *reinterpret_cast<uint4*>(tile_base + tile_off<D>(in_page, chunk)) = v;
        }
        __syncthreads();
        uint32_t qa[KS][4];
#pragma unroll
        for (int kk = 0; kk < KS; ++kk)
            ldmatrix_x4(qa[kk], q_s + swz<D>(lane & 15, kk * 2 + (lane >> 4)));

        const float sc = scale * kLog2e;
        for (int it = warp; it < count; it += kClWarps) {
            // the whole warp leaves together if any lane's wait ran out
            if (!__all_sync(0xffffffffu, mbar_wait(bars + it, 0))) {
                failed = true;
                break;
            }
            const bf16* kt = tiles + (size_t)it * 2 * TILE;
            const bf16* vt = kt + TILE;
            const int t_page = (begin + it) * kClPage;

            // scores of the page's 64 keys in four groups of 16: S[16 heads, 16 keys] = Q . K^T
            float s[4][2][4];
#pragma unroll
            for (int g = 0; g < 4; ++g) {
                const int key0 = g * 16;
#pragma unroll
                for (int j = 0; j < 2; ++j)
#pragma unroll
                    for (int e = 0; e < 4; ++e) s[g][j][e] = 0.f;
                uint32_t kb[KS / 2][2][4];
#pragma unroll
                for (int kk = 0; kk < KS; kk += 2)
#pragma unroll
                    for (int j = 0; j < 2; ++j)
                        // four 8x8 tiles: keys j*8.., dims kk*16 .. kk*16+31
                        ldmatrix_x4(kb[kk / 2][j],
                                    kt + tile_off<D>(key0 + j * 8 + (lane & 7), kk * 2 + (lane >> 3)));
#pragma unroll
                for (int kk = 0; kk < KS; kk += 2) {
#pragma unroll
                    for (int j = 0; j < 2; ++j) {
                        mma_bf16(s[g][j], qa[kk], kb[kk / 2][j][0], kb[kk / 2][j][1]);
                        mma_bf16(s[g][j], qa[kk + 1], kb[kk / 2][j][2], kb[kk / 2][j][3]);
                    }
                }
            }
            // mask, scale (in log2 units) and the page's row maxima
            float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
            for (int g = 0; g < 4; ++g)
#pragma unroll
                for (int j = 0; j < 2; ++j)
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        int t = t_page + g * 16 + j * 8 + c_lo + (e & 1);
                        float v = (t >= lo && t < hi) ? s[g][j][e] * sc : -INFINITY;
                        s[g][j][e] = v;
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
            uint32_t pa[4][4];
            float psum[2] = {0.f, 0.f};
#pragma unroll
            for (int g = 0; g < 4; ++g)
#pragma unroll
                for (int j = 0; j < 2; ++j) {
                    float p0v = exp2f(s[g][j][0] - base[0]), p1v = exp2f(s[g][j][1] - base[0]);
                    float p2v = exp2f(s[g][j][2] - base[1]), p3v = exp2f(s[g][j][3] - base[1]);
                    psum[0] += p0v + p1v;
                    psum[1] += p2v + p3v;
                    pa[g][j * 2] = pack_bf16(p0v, p1v);
                    pa[g][j * 2 + 1] = pack_bf16(p2v, p3v);
                }
#pragma unroll
            for (int r = 0; r < 2; ++r) l_run[r] = l_run[r] * alpha[r] + psum[r];
            // output: O = O * alpha + P . V, the page's four groups of 16 keys one after another
#pragma unroll
            for (int jn = 0; jn < NT; jn += 2) {
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    o[jn][e] *= alpha[e >> 1];
                    o[jn + 1][e] *= alpha[e >> 1];
                }
                uint32_t vb[4][4];
#pragma unroll
                for (int g = 0; g < 4; ++g)
                    // keys 0-7 / 8-15 of the group, dims jn*8 .. jn*8+15
                    ldmatrix_x4_trans(vb[g], vt + tile_off<D>(g * 16 + (lane & 15), jn + (lane >> 4)));
#pragma unroll
                for (int g = 0; g < 4; ++g) {
                    mma_bf16(o[jn], pa[g], vb[g][0], vb[g][1]);
                    mma_bf16(o[jn + 1], pa[g], vb[g][2], vb[g][3]);
                }
            }
        }
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 1);
            l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 2);
        }
    }
    if (failed && lane == 0 && status) atomicExch(status, 2);
    // A warp that gave up must not leave copies in flight behind it: wait (bounded
    // again) for every page that was asked for before shared memory is given up.
    if (__syncthreads_or(failed) && tid == 0)
        for (int it = 0; it < count; ++it) mbar_wait(bars + it, 0);
    __syncthreads();  // everyone is done with the tiles: reuse them for the merge
    trace_mark(trace, 4);
    trace_mark(trace, 5);
    // The same pages of the cache that is read next (`ahead` elements on: the next layer
    // of the group) are asked into L2 now: its kernel starts some ten microseconds on.
    if (ahead != 0 && tid < count) {
        const size_t row0 = (size_t)(ids[begin - p0 + tid] * nkv + hk) * kClPage;
        l2_prefetch(k_cache + ahead + row0 * D, TILE * (uint32_t)sizeof(bf16));
        l2_prefetch(v_cache + ahead + row0 * D, TILE * (uint32_t)sizeof(bf16));
    }

    // ---- merge the four warps: (m, l) through sm_ml, outputs through the tiles ----
    float* o_s = reinterpret_cast<float*>(tiles);                  // [warps, 16, D] float32
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
    for (int item = tid; item < gcount * CH; item += kClThreads) {
        int row = item / CH, chunk = item % CH;
        float mm = -INFINITY;
#pragma unroll
        for (int w = 0; w < kClWarps; ++w) mm = fmaxf(mm, sm_ml[w][row][0]);
        float ll = 0.f, acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        if (mm != -INFINITY) {
#pragma unroll
            for (int w = 0; w < kClWarps; ++w) {
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
    // One thread takes the ticket with release and acquire in the one instruction: after
    // the barrier its release also covers what the other threads of the CTA wrote, and
    // what the last one reads after the next barrier comes after the others' releases.
    __syncthreads();
    unsigned* ticket = tickets + ((size_t)n * nkv + hk) * head_tiles + tile;
    if (tid == 0) is_last = ticket_take(ticket) == (unsigned)n_splits - 1u;
    __syncthreads();
    trace_mark(trace, 6);
    trace_mark(trace, 7);
    if (!is_last) {
        trace_mark(trace, 1);
        return;
    }
    // One trip to L2: a thread owns (row, 8 dims, one of four interleaved groups of
    // slices) and asks for the maxima, sums and outputs of its slices all at once;
    // it folds them against the group's own maximum, and the four groups of a row
    // meet in shared memory, added in the order of the groups.
    float* g_ml = &sm_ml[0][0][0];   // [4, 16, 2] group maximum and sum
    float* g_o = o_s;                // [4, 16, D] group outputs
    constexpr int kRound = 4;  // slices of a group asked for at once (all of them up to 16 slices)
    for (int item = tid; item < gcount * CH * 4; item += kClThreads) {
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
    for (int item = tid; item < gcount * CH; item += kClThreads) {
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
static size_t tma_smem_bytes(int per) {
    size_t q_bytes = 16 * (size_t)D * sizeof(bf16);
    size_t page_bytes = (size_t)per * 2 * kClPage * D * sizeof(bf16);
    size_t merge_bytes = (size_t)kClWarps * 16 * D * sizeof(float);
    return q_bytes + (page_bytes < merge_bytes ? merge_bytes : page_bytes);
}

// pages of one slice that fit the shared memory of a CTA beside the query rows
static int tma_max_pages(int d) {
    const size_t limit = 227 * 1024;
    int pages = (int)((limit - 16 * (size_t)d * sizeof(bf16)) / (2 * (size_t)kClPage * d * sizeof(bf16)));
    return pages < kMaxPages ? pages : kMaxPages;
}

template <int D>
static int launch_tma(dim3 grid, int per, bool pdl, cudaStream_t stream, const CUtensorMap& mk,
                      const CUtensorMap& mv, const bf16* k_cache, const bf16* v_cache, const bf16* q,
                      int q_stride, const int* pos, const int* seq, const int* table, int cols,
                      bf16* out, float* partial, unsigned* tickets, int nq, int nkv, int window,
                      float scale, int head_tiles, int* status, long long ahead) {
    const size_t smem = tma_smem_bytes<D>(per);
    auto kernel = attn_decode_tma_kernel<D>;
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(kClThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 1 : 0;
    e = cudaLaunchKernelEx(&cfg, kernel, mk, mv, k_cache, v_cache, q, q_stride, pos, seq, table, cols,
                           out, partial, tickets, nq, nkv, window, scale, (int)grid.z, head_tiles, per,
                           status, ahead, trace_slot("attention decode (tma)"));
    return e == cudaSuccess ? NNIS_OK : (int)e;
}

// How many CTAs of this kernel, each holding `per` pages, one SM runs at once.
template <int D>
static int tma_ctas_per_sm(int per) {
    auto kernel = attn_decode_tma_kernel<D>;
    const size_t smem = tma_smem_bytes<D>(per);
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
        return 0;
    int blocks = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&blocks, kernel, kClThreads, smem) != cudaSuccess) {
        (void)cudaGetLastError();
        return 0;
    }
    return blocks;
}

}  // namespace nnis

// The most pages per slice for head size `d` (0: head size not taken).
NNIS_API int nnis_attention_decode_tma_max_pages(int d) {
    return d == 64 || d == 128 ? nnis::tma_max_pages(d) : 0;
}

// CTAs of `per` pages that one SM runs at once for head size `d` (0: not possible).
NNIS_API int nnis_attention_decode_tma_ctas_per_sm(int d, int per) {
    if ((d != 64 && d != 128) || per < 1 || per > nnis::tma_max_pages(d)) return 0;
    return d == 64 ? nnis::tma_ctas_per_sm<64>(per) : nnis::tma_ctas_per_sm<128>(per);
}

// One query token per sequence over the paged bfloat16 cache; the key range of a
// sequence (table_cols pages) is cut into n_splits slices of ceil(table_cols / n_splits)
// pages, at most 8 pages a slice (6 at head size 128).  Scratch as for
// nnis_attention_decode_mma: with n_splits > 1, `partial` (n_tokens * nq * n_splits *
// (d + 2) floats) and `tickets` (n_tokens * nkv * ceil(group / 16) counters, zero before
// the first launch; the kernel leaves them zero).  `cache_rows`: pages x kv heads x 64,
// the rows of the cache seen as a matrix of head_dim columns.  `ahead`: elements from these
// caches to the ones that are read next (the next layer's), whose same pages this kernel
// asks into L2; 0: none.
NNIS_API int nnis_attention_decode_tma(const void* q, int q_stride, const void* k_cache,
                                       const void* v_cache, long long cache_rows,
                                       const int* token_pos, const int* token_seq,
                                       const int* page_table, int table_cols, void* out,
                                       float* partial, unsigned* tickets, int n_tokens, int nq,
                                       int nkv, int d, int page_size, int window, float scale,
                                       int n_splits, long long ahead, int* status, int pdl,
                                       cudaStream_t stream) {
    using namespace nnis;
    if (n_tokens <= 0 || nq <= 0 || nkv <= 0 || nq % nkv || table_cols <= 0 || n_splits <= 0 ||
        window < 0 || cache_rows <= 0)
        return NNIS_ERR_ARGUMENT;
    if ((d != 64 && d != 128) || page_size != kClPage) return NNIS_ERR_UNSUPPORTED;
    const int per = (table_cols + n_splits - 1) / n_splits;
    if (n_tokens > 65535 || n_splits > kMaxSlices || per > tma_max_pages(d) || cache_rows >= (1ll << 31))
        return NNIS_ERR_UNSUPPORTED;
    if (n_splits > 1 && (!partial || !tickets)) return NNIS_ERR_ARGUMENT;
    if (((uintptr_t)q | (uintptr_t)k_cache | (uintptr_t)v_cache | (uintptr_t)out) % 16 ||
        (q_stride % 8))
        return NNIS_ERR_ALIGNMENT;
    CUtensorMap mk, mv;
    if (!make_map(&mk, k_cache, cache_rows, d, kClPage) || !make_map(&mv, v_cache, cache_rows, d, kClPage))
        return NNIS_ERR_UNSUPPORTED;
    int G = nq / nkv;
    int head_tiles = (G + 15) / 16;
    dim3 grid(nkv * head_tiles, n_tokens, n_splits);
    if (d == 64)
        return launch_tma<64>(grid, per, pdl != 0, stream, mk, mv, (const bf16*)k_cache,
                              (const bf16*)v_cache, (const bf16*)q, q_stride, token_pos, token_seq,
                              page_table, table_cols, (bf16*)out, partial, tickets, nq, nkv, window,
                              scale, head_tiles, status, ahead);
    return launch_tma<128>(grid, per, pdl != 0, stream, mk, mv, (const bf16*)k_cache,
                           (const bf16*)v_cache, (const bf16*)q, q_stride, token_pos, token_seq,
                           page_table, table_cols, (bf16*)out, partial, tickets, nq, nkv, window, scale,
                           head_tiles, status, ahead);
}
