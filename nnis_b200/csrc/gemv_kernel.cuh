// (Kernel and launch templates; gemv_bf16.cu holds the entry point and gemv_tiles*.cu
// the instantiations, one file per number of row tiles, so that they compile side by side.)
//
// Projections of a decode step in bfloat16: y[M, N] = x[M, K] . W[N, K]^T with
// at most 64 rows of x.  The step is bound by the bytes of W and by latency, so
//
//  * W is brought into shared memory by bulk asynchronous copies (one per
//    weight row, completing on an mbarrier), issued before anything else in the
//    kernel - before the wait of programmatic dependent launch, hence while the
//    kernel before it still runs - and double-buffered per warp where that pays;
//  * the products run on the tensor cores (mma.sync m16n8k16, float32
//    accumulation): x is the 16-row A operand (one to four tiles of rows), eight
//    weight rows are the B operand, so a warp needs about a hundred instructions
//    per eight outputs instead of a thousand on the CUDA cores, and no reduction
//    across lanes;
//  * what surrounds the product is fused so that no activation makes a round
//    trip through its own kernel:
//      prologue  NORM:  x = bf16(rmsnorm(hidden_f32[rows]) * w_norm);
//      epilogue  STORE (bfloat16), STORE_F32, ADD_F32 (into the residual stream),
//                GATED:  out[m, i] = bf16(silu(y[m, i]) * y[m, I + i]),
//                QKV:    bias, round, rotate-half RoPE of q and k heads at each
//                        row's position, q to a packed buffer, k and v into the
//                        paged cache,
//                ARGMAX: the index of the largest y per row (ties to the lower
//                        index), optionally the float32 logits too, and the move
//                        of the decode state to the next token.
//
// A warp owns eight output rows at a time (a "unit").  Shared-memory rows are
// padded by 16 bytes so that ldmatrix meets no bank conflict when K is a multiple
// of 16.  NNIS's one-token projection: crates/nnis-kernels/src/gemv.rs:45-61; its
// fused gate/up/SiLU kernel: crates/nnis-model/src/fused_swiglu.rs:14-27; its
// greedy pick: crates/nnis-kernels/src/top_k.rs:57-70.
#include <float.h>

#pragma once

#include "mma_helpers.cuh"

namespace nnis {

enum { EPI_STORE = 0, EPI_STORE_F32 = 1, EPI_ADD_F32 = 2, EPI_GATED = 3, EPI_QKV = 4, EPI_ARGMAX = 5 };
// PRO_SCALED (gemv_rowtile.cu only): x is bf16(h * w_norm), what an ADD_F32 epilogue before
// this kernel emitted with its shares of each row's sum of squares; the rows' scales
// 1 / sqrt(mean of squares + eps) are applied to the float32 sums, after the products.
enum { PRO_PLAIN = 0, PRO_NORM = 1, PRO_SCALED = 2 };

struct GemvArgs {
    const bf16* x;          // [M, K] (plain prologue)
    const float* hidden;    // [*, K] float32 residual stream (norm prologue)
    const int* rows;        // optional row of `hidden` per x row
    const float* norm_w;    // [K]
    float eps;
    const bf16* w;          // [N, K]
    const float* bias;      // [N] or null
    void* out;              // see epilogues
    int M, N, K;
    int ldx, ldw;           // elements between rows of x and of w (K unless a slice of K is taken)
    int kc;                 // columns of K per weight stage (K: a stage holds whole rows)
    int out_is_hot;         // ADD_F32: the kernel just before this one wrote `out` (a slice of K)
    int release_early;      // the kernel after this one may start at once (see below)
    int* status;            // set non-zero when a bounded wait runs out
    // QKV epilogue
    const int* token_pos;
    const int* token_seq;
    const int* page_table;
    int table_cols;
    const float* cos_t;
    const float* sin_t;     // null: no rotation
    bf16* k_cache;
    bf16* v_cache;
    int nq, nkv, d, page_size;
    // ARGMAX epilogue
    float* logits;          // optional [M, N]
    float* best_val;        // [M, gridDim.x]
    int* best_idx;          // [M, gridDim.x]
    unsigned* ticket;       // one counter, zero between launches
    int* next_tokens;       // optional: tokens of the next step (picked) ...
    int* next_pos;          // ... and their positions (+1 on live rows)
    unsigned long long* trace;  // this launch's slot of the step's timeline, or null
    // ADD_F32 epilogue, optional: the norm that follows this projection, begun here.  For
    // every value of the residual stream that it has just summed the epilogue also writes
    // bf16(value * emit_w[column]) to emit_x [M, N] and, per unit of eight columns and row,
    // the sum of the eight squares to emit_ss [M, N / 8].
    bf16* emit_x;
    const float* emit_w;
    float* emit_ss;
    // PRO_SCALED prologue: those shares of the rows' sums of squares, [M, ss_units]
    const float* ss_parts;
    int ss_units;
};

__device__ __forceinline__ float round_bf16(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }

__device__ __forceinline__ bool better(float v, int i, float bv, int bi) {
    return bi < 0 || v > bv || (v == bv && i < bi);
}

__device__ __forceinline__ void ldmatrix_x2(uint32_t& r0, uint32_t& r1, const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0,%1}, [%2];"
                 : "=r"(r0), "=r"(r1)
                 : "r"(smem_addr(p)));
}

// Output row of column c (0..7) of unit `unit`: columns 0-3 and 4-7 are the two
// halves of a pair in the GATED (gate, up) and QKV (j, j + d/2) epilogues.
template <int EPI>
__device__ __forceinline__ int unit_row(const GemvArgs& a, int unit, int c) {
    if (EPI == EPI_GATED) return (c < 4 ? 0 : (a.N >> 1) - 4) + unit * 4 + c;
    if (EPI == EPI_QKV) {
        int per_head = a.d >> 3;
        int head = unit / per_head, jj = (unit - head * per_head) * 4;
        return head * a.d + jj + (c < 4 ? c : (a.d >> 1) + c - 4);
    }
    return unit * 8 + c;
}

// The norm prologue for rows too long for a lane's registers, in two passes over the
// row, each with eight loads in flight per lane (a loop of single loads would wait for L2
// once per iteration).  A lane takes the float4 at `first`, `first` + STRIDE, ...
template <int STRIDE>
__device__ __forceinline__ float row_square_sum(const float4* h4, int k4, int first) {
    float ss = 0.f;
    for (int c0 = first; c0 < k4; c0 += STRIDE * 8) {
        float4 v[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            int c = c0 + STRIDE * j;
            v[j] = c < k4 ? h4[c] : make_float4(0.f, 0.f, 0.f, 0.f);
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            ss = fmaf(v[j].x, v[j].x, ss);
            ss = fmaf(v[j].y, v[j].y, ss);
            ss = fmaf(v[j].z, v[j].z, ss);
            ss = fmaf(v[j].w, v[j].w, ss);
        }
    }
    return ss;
}

// ... and the row scaled by `sc`, weighted and rounded to bfloat16 at `dst`.
template <int STRIDE>
__device__ __forceinline__ void row_scale_store(const float4* h4, const float4* w4, int k4, int first,
                                                float sc, bf16* dst) {
    for (int c0 = first; c0 < k4; c0 += STRIDE * 8) {
        float4 v[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            int c = c0 + STRIDE * j;
            v[j] = c < k4 ? h4[c] : make_float4(0.f, 0.f, 0.f, 0.f);
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            int c = c0 + STRIDE * j;
            if (c < k4) {
                const float4 g = w4[c];
                store4(dst + c * 4, make_float4((v[j].x * sc) * g.x, (v[j].y * sc) * g.y,
                                                (v[j].z * sc) * g.z, (v[j].w * sc) * g.w));
            }
        }
    }
}

// What the epilogue of one tile of 16 rows needs from global memory and that no product
// decides: fetched before the wait of programmatic dependent launch (the residual stream
// was last written two kernels back, positions and page tables before the step began).
// A lane holds rows r_lo = lane / 4 and r_lo + 8 of the tile, columns c_lo = 2 (lane % 4)
// and c_lo + 1 of the unit.
struct EpiTile {
    float2 old[2];                  // ADD_F32: the destination's values (first unit only)
    int pos[2], page[2];            // QKV: the rows' positions and cache pages
    float cs[4], sn[4];             // QKV: the rotation at those positions (first unit only)
    float2 ew;                      // ADD_F32 that emits: the next norm's weights (first unit only)
};

// QKV: where a head's values go.  Row m of a query head lies at base + m * row_step (the
// packed q rows); a row of a key or value head at base + place * row_step + page * page_step
// (its place in the head's part of its cache page).
template <int EPI>
__device__ __forceinline__ void qkv_head(const GemvArgs& a, int head, bf16*& base, size_t& row_step,
                                         size_t& page_step) {
    if (head < a.nq) {
        base = reinterpret_cast<bf16*>(a.out) + (size_t)head * a.d;
        row_step = (size_t)a.nq * a.d;
        page_step = 0;
    } else {
        const bool is_v = head >= a.nq + a.nkv;
        const int hk = is_v ? head - a.nq - a.nkv : head - a.nq;
        base = (is_v ? a.v_cache : a.k_cache) + (size_t)hk * a.page_size * a.d;
        row_step = (size_t)a.d;
        page_step = (size_t)a.nkv * a.page_size * a.d;
    }
}

// `every_unit`: the warp goes on to other units with what it fetched for the rows (else
// the cache page of a row is looked up only if this unit is of a key or value head).
template <int EPI>
__device__ __forceinline__ void epi_preload(const GemvArgs& a, int unit, int row0, int lane, bool every_unit,
                                            EpiTile& p) {
    const int r_lo = lane >> 2, c_lo = (lane & 3) * 2;
    if (EPI == EPI_ADD_F32 && !a.out_is_hot) {
        const int n0 = unit * 8 + c_lo;
#pragma unroll
        for (int hrow = 0; hrow < 2; ++hrow) {
            int m = row0 + r_lo + hrow * 8;
            p.old[hrow] = m < a.M ? *reinterpret_cast<const float2*>(
                                        reinterpret_cast<const float*>(a.out) + (size_t)m * a.N + n0)
                                  : make_float2(0.f, 0.f);
        }
    }
    if (EPI == EPI_ADD_F32 && a.emit_x)
        p.ew = *reinterpret_cast<const float2*>(a.emit_w + unit * 8 + c_lo);
    if (EPI == EPI_QKV) {
        const int na = unit_row<EPI>(a, unit, c_lo & 3);
        const int head = na / a.d, j = na - head * a.d, hf = a.d >> 1;
        const bool rotate = a.sin_t && head < a.nq + a.nkv;
        const bool paged = a.nkv > 0 && (every_unit || head >= a.nq);
#pragma unroll
        for (int hrow = 0; hrow < 2; ++hrow) {
            int m = row0 + r_lo + hrow * 8;
            int pos = m < a.M ? a.token_pos[m] : -1;
            p.pos[hrow] = pos;
            // (the row's page holds for every unit)
            p.page[hrow] = pos >= 0 && paged
                               ? a.page_table[(size_t)a.token_seq[m] * a.table_cols + pos / a.page_size] : 0;
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                p.cs[hrow * 2 + e] = (rotate && pos >= 0) ? a.cos_t[(size_t)pos * hf + j + e] : 1.f;
                p.sn[hrow * 2 + e] = (rotate && pos >= 0) ? a.sin_t[(size_t)pos * hf + j + e] : 0.f;
            }
        }
    }
}

// The epilogue of one tile of 16 rows of one unit: `v` are this lane's four sums
// (rows r_lo, r_lo + 8 x columns c_lo, c_lo + 1).  `first`: p.old, p.cs and p.sn were
// fetched for this unit.  Every lane of the warp must call it (the halves of a pair
// change hands by shuffle).  ARGMAX keeps the best of the lane's columns per row.
template <int EPI>
__device__ __forceinline__ void epi_finish(const GemvArgs& a, int unit, int row0, int lane,
                                           const float (&v)[4], const EpiTile& p, bool first,
                                           float (&best_v)[2], int (&best_i)[2]) {
    const int r_lo = lane >> 2, c_lo = (lane & 3) * 2;
    const int M = a.M;
    if (EPI == EPI_GATED || EPI == EPI_QKV) {
        // columns 0-3 pair with 4-7: the lanes of the second half hand theirs over
        const bool low = (lane & 3) < 2;
        const int n_a = unit_row<EPI>(a, unit, c_lo & 3);  // even: this lane finishes n_a, n_a + 1
        const int n_b = unit_row<EPI>(a, unit, (c_lo & 3) + 4);
        float pv[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) pv[e] = __shfl_xor_sync(0xffffffffu, v[e], 2);
        if (!low) return;
        float bias_a[2] = {0.f, 0.f}, bias_b[2] = {0.f, 0.f};
        if (a.bias) {
            bias_a[0] = a.bias[n_a]; bias_a[1] = a.bias[n_a + 1];
            bias_b[0] = a.bias[n_b]; bias_b[1] = a.bias[n_b + 1];
        }
        // QKV: what the unit decides (a unit lies inside one head)
        const int half = a.d >> 1, inter = a.N >> 1;
        int head = 0, j = 0;
        bf16* base = nullptr;
        size_t row_step = 0, page_step = 0;
        if (EPI == EPI_QKV) {
            head = n_a / a.d;
            j = n_a - head * a.d;
            qkv_head<EPI>(a, head, base, row_step, page_step);
        }
        const bool rotate = EPI == EPI_QKV && a.sin_t && head < a.nq + a.nkv;
#pragma unroll
        for (int hrow = 0; hrow < 2; ++hrow) {
            int m = row0 + r_lo + hrow * 8;
            if (m >= M) continue;
            float va[2], vb[2];
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                va[e] = v[hrow * 2 + e] + bias_a[e];
                vb[e] = pv[hrow * 2 + e] + bias_b[e];
            }
            if (EPI == EPI_GATED) {
                *reinterpret_cast<uint32_t*>(reinterpret_cast<bf16*>(a.out) + (size_t)m * inter + n_a) =
                    pack_bf16((va[0] / (1.0f + expf(-va[0]))) * vb[0],
                              (va[1] / (1.0f + expf(-va[1]))) * vb[1]);
            } else {
                int pos = p.pos[hrow];
                if (pos < 0) continue;
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    va[e] = round_bf16(va[e]);
                    vb[e] = round_bf16(vb[e]);
                    if (rotate) {
                        float c = first ? p.cs[hrow * 2 + e] : a.cos_t[(size_t)pos * half + j + e];
                        float sn = first ? p.sn[hrow * 2 + e] : a.sin_t[(size_t)pos * half + j + e];
                        float ra = va[e] * c - vb[e] * sn, rb = vb[e] * c + va[e] * sn;
                        va[e] = ra;
                        vb[e] = rb;
                    }
                }
                bf16* o = head < a.nq ? base + (size_t)m * row_step
                                      : base + (size_t)(pos % a.page_size) * row_step +
                                            (size_t)p.page[hrow] * page_step;
                *reinterpret_cast<uint32_t*>(o + j) = pack_bf16(va[0], va[1]);
                *reinterpret_cast<uint32_t*>(o + j + half) = pack_bf16(vb[0], vb[1]);
            }
        }
    } else {
        const int n0 = unit * 8 + c_lo;
        const float b0v = a.bias ? a.bias[n0] : 0.f, b1v = a.bias ? a.bias[n0 + 1] : 0.f;
        float emit_sq[2] = {0.f, 0.f};  // ADD_F32 that emits: this lane's two squares of each row
        float2 ew = make_float2(0.f, 0.f);
        if (EPI == EPI_ADD_F32 && a.emit_x) ew = first ? p.ew : *reinterpret_cast<const float2*>(a.emit_w + n0);
#pragma unroll
        for (int hrow = 0; hrow < 2; ++hrow) {
            int m = row0 + r_lo + hrow * 8;
            if (m >= M) continue;
            float v0 = v[hrow * 2] + b0v, v1 = v[hrow * 2 + 1] + b1v;
            size_t o = (size_t)m * a.N + n0;
            if (EPI == EPI_STORE) {
                *reinterpret_cast<uint32_t*>(reinterpret_cast<bf16*>(a.out) + o) = pack_bf16(v0, v1);
            } else if (EPI == EPI_STORE_F32) {
                *reinterpret_cast<float2*>(reinterpret_cast<float*>(a.out) + o) = make_float2(v0, v1);
            } else if (EPI == EPI_ADD_F32) {
                float2* q = reinterpret_cast<float2*>(reinterpret_cast<float*>(a.out) + o);
                float2 old = (first && !a.out_is_hot) ? p.old[hrow] : *q;
                const float2 sum = make_float2(old.x + v0, old.y + v1);
                *q = sum;
                if (a.emit_x) {
                    *reinterpret_cast<uint32_t*>(a.emit_x + o) =
                        pack_bf16(sum.x * ew.x, sum.y * ew.y);
                    emit_sq[hrow] = fmaf(sum.x, sum.x, sum.y * sum.y);
                }
            } else {
                if (a.logits) *reinterpret_cast<float2*>(a.logits + o) = make_float2(v0, v1);
                if (better(v0, n0, best_v[hrow], best_i[hrow])) {
                    best_v[hrow] = v0;
                    best_i[hrow] = n0;
                }
                if (better(v1, n0 + 1, best_v[hrow], best_i[hrow])) {
                    best_v[hrow] = v1;
                    best_i[hrow] = n0 + 1;
                }
            }
        }
        if (EPI == EPI_ADD_F32 && a.emit_x) {  // (uniform over the warp: every lane shuffles)
#pragma unroll
            for (int hrow = 0; hrow < 2; ++hrow) {
                // the four lanes of a row, in lane order: columns 0-1, 2-3, 4-5, 6-7
                float sq = emit_sq[hrow];
                sq += __shfl_xor_sync(0xffffffffu, sq, 1);
                sq += __shfl_xor_sync(0xffffffffu, sq, 2);
                int m = row0 + r_lo + hrow * 8;
                if ((lane & 3) == 0 && m < M) a.emit_ss[(size_t)m * (a.N >> 3) + unit] = sq;
            }
        }
    }
}

// MTILES tiles of 16 rows of x; WARPS warps per CTA; S stages of weights per warp.
// SPLITK: the CTA owns one unit and its warps share K (each a run of 16-column
// steps), which shortens the chain of dependent products when there are fewer
// units than the GPU has room for; the partial sums meet in shared memory and
// warp 0 adds them in order and runs the epilogue.
template <int MTILES, int EPI, int PRO, int S, int WARPS, bool SPLITK>
__global__ void __launch_bounds__(WARPS * 32)
gemv_kernel(GemvArgs a) {
    constexpr int MT = MTILES * 16;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    trace_mark(a.trace, 0);
    // A caller that knows what runs next may let it start with this kernel instead of
    // after this kernel's wait: it must be a kernel that reads, before its own wait,
    // nothing that any kernel of the step writes (the decode attention reads positions,
    // page ids and old cache pages there), and that releases its own dependents only
    // after its wait, so that kernels further on still find everything before their
    // immediate predecessor complete.
    if (a.release_early) pdl_launch_dependents();
    const int K = a.K, M = a.M;
    const int KP = K + 8;  // padded row, in elements
    // A weight stage holds eight rows of KC columns: all of K, or with long rows a
    // chunk of it, so that a warp still has a stage in flight while it multiplies.
    const int KC = SPLITK ? K : a.kc;
    const int KCP = KC + 8;
    const int n_chunks = SPLITK ? 1 : (K + KC - 1) / KC;
    bf16* xs = reinterpret_cast<bf16*>(smem_raw);                          // [MT, KP]
    // weight stages: one set per warp, or one shared set when the warps split K
    bf16* wst = xs + (size_t)MT * KP + (SPLITK ? 0 : (size_t)warp * S * 8 * KCP);
    constexpr int kSets = SPLITK ? 1 : WARPS * S;
    uint64_t* bars = reinterpret_cast<uint64_t*>(xs + (size_t)MT * KP + (size_t)kSets * 8 * KCP) + warp * S;
    float* red = reinterpret_cast<float*>(bars - warp * S + WARPS * S);     // SPLITK: [WARPS, MTILES*4, 32]
    __shared__ float cta_val[WARPS][MT];
    __shared__ int cta_idx[WARPS][MT];
    __shared__ bool is_last;
    __shared__ __align__(8) uint64_t xbar;  // the bulk copies of x complete here

    const int n_units = a.N >> 3;
    const int unit_stride = SPLITK ? gridDim.x : gridDim.x * WARPS;
    // units are dealt to CTAs first, so that few units still spread over many SMs
    const int first_unit = SPLITK ? blockIdx.x : warp * gridDim.x + blockIdx.x;
    // this warp's columns of K: all of them, or its share of the 16-column steps
    const int steps = K >> 4;
    const int steps_per_warp = (steps + WARPS - 1) / WARPS;
    const int k_begin = SPLITK ? min(steps, warp * steps_per_warp) * 16 : 0;
    const int k_end = SPLITK ? min(steps, (warp + 1) * steps_per_warp) * 16 : K;
    const uint32_t row_bytes = (uint32_t)(k_end - k_begin) * 2u;
    // With the warps sharing K, one tile of rows and x as it is (no norm), a warp needs
    // only its own columns of x and takes them from global memory straight into the
    // registers of its products: no trip of x through shared memory, no barrier for it.
    // (The same with the norm in front, the warps exchanging their shares of each row's
    // sum of squares, was measured slower: its registers keep the next kernel's CTAs
    // from becoming resident early.)
    constexpr bool kDirect = SPLITK && PRO == PRO_PLAIN && MTILES == 1;
    // 16-column steps of one warp: K <= 1,536 with eight warps
    constexpr int kDirectSteps = kDirect ? 12 : 1;
    const bool direct = kDirect && steps_per_warp <= kDirectSteps;
    uint32_t ax[kDirectSteps][4];

    // stage j holds chunk j % n_chunks of this warp's unit number j / n_chunks
    auto issue = [&](int j) {  // lane 0 only
        const int i = n_chunks == 1 ? j : j / n_chunks;
        const int unit = first_unit + i * unit_stride;
        if (unit >= n_units) return;
        const int kc0 = SPLITK ? k_begin : (j - i * n_chunks) * KC;
        const uint32_t bytes = SPLITK ? row_bytes : (uint32_t)min(KC, K - kc0) * 2u;
        if (bytes == 0) return;
        uint64_t* bar = bars + (j % S);
        bf16* dst = wst + (size_t)(j % S) * 8 * KCP + (SPLITK ? k_begin : 0);
        mbar_expect_tx(bar, 8u * bytes);
#pragma unroll
        for (int c = 0; c < 8; ++c)
            bulk_load(dst + (size_t)c * KCP, a.w + (size_t)unit_row<EPI>(a, unit, c) * a.ldw + kc0,
                      bytes, bar);
    };

    // ---- weights first: they depend on no earlier kernel ---------------------
    if (lane == 0) {
#pragma unroll
        for (int s = 0; s < S; ++s) mbar_init(bars + s, 1);
        if (warp == 0) mbar_init(&xbar, 1);
        mbar_fence_init();
#pragma unroll
        for (int s = 0; s < S; ++s) issue(s);
    }
    // ... and the norm weights of this lane's columns
    constexpr int NW = 6;  // float4 per lane kept in registers: covers K <= 768
    float4 nw[NW];
    const int k4 = K >> 2;
    if (PRO == PRO_NORM) {
#pragma unroll
        for (int j = 0; j < NW; ++j) {
            int c = lane + 32 * j;
            nw[j] = c < k4 ? reinterpret_cast<const float4*>(a.norm_w)[c] : make_float4(0.f, 0.f, 0.f, 0.f);
        }
    }
    // What the epilogue of this warp's first unit needs from global memory does not
    // come from the kernel just before this one either, so it is fetched now, under that
    // kernel's tail, instead of after the products.
    const int r_lo = lane >> 2;
    // A warp finishes all tiles of rows of its own units; with the warps sharing K,
    // warp t finishes tile t of the CTA's unit (the sums and the epilogue of the tiles
    // then run side by side instead of in one warp).
    constexpr int ET = SPLITK ? 1 : MTILES;
    const bool epi_warp = !SPLITK || warp < MTILES;
    auto tile_of = [&](int tt) { return SPLITK ? warp : tt; };
    EpiTile pre[ET];
    if (epi_warp && first_unit < n_units) {
#pragma unroll
        for (int tt = 0; tt < ET; ++tt) epi_preload<EPI>(a, first_unit, tile_of(tt) * 16, lane, !SPLITK, pre[tt]);
    }
    // Dependents are released only after this kernel's own wait: a kernel that
    // starts early may then rely on everything before its immediate predecessor
    // (the decode attention kernel reads old cache pages before its wait).
    if (PRO == PRO_PLAIN) __syncthreads();  // every warp sees the barrier of x initialised
    pdl_wait();
    if (!a.release_early) pdl_launch_dependents();

    trace_mark(a.trace, 2);
    trace_mark(a.trace, 3);

    bool failed = false;
    // ---- x into shared memory (or, see above, straight into registers) ---------
    if (PRO == PRO_NORM) {
        const bool in_regs = k4 <= 32 * NW;
        for (int m = warp; m < MT; m += WARPS) {
            if (m < M) {
                const float* h = a.hidden + (size_t)(a.rows ? a.rows[m] : m) * K;
                const float4* h4 = reinterpret_cast<const float4*>(h);
                float4 hv[NW];
                float ss = 0.f;
                if (in_regs) {
#pragma unroll
                    for (int j = 0; j < NW; ++j) {
                        int c = lane + 32 * j;
                        hv[j] = c < k4 ? h4[c] : make_float4(0.f, 0.f, 0.f, 0.f);
                    }
#pragma unroll
                    for (int j = 0; j < NW; ++j) {
                        ss = fmaf(hv[j].x, hv[j].x, ss);
                        ss = fmaf(hv[j].y, hv[j].y, ss);
                        ss = fmaf(hv[j].z, hv[j].z, ss);
                        ss = fmaf(hv[j].w, hv[j].w, ss);
                    }
                } else {
                    for (int c = lane; c < k4; c += 32) {
                        float4 v = h4[c];
                        ss = fmaf(v.x, v.x, ss);
                        ss = fmaf(v.y, v.y, ss);
                        ss = fmaf(v.z, v.z, ss);
                        ss = fmaf(v.w, v.w, ss);
                    }
                }
                ss = warp_sum(ss);
                float s = 1.0f / sqrtf(ss * (1.0f / (float)K) + a.eps);
                if (in_regs) {
#pragma unroll
                    for (int j = 0; j < NW; ++j) {
                        int c = lane + 32 * j;
                        if (c < k4) {
                            float4 r = make_float4((hv[j].x * s) * nw[j].x, (hv[j].y * s) * nw[j].y,
                                                   (hv[j].z * s) * nw[j].z, (hv[j].w * s) * nw[j].w);
                            store4(xs + (size_t)m * KP + c * 4, r);
                        }
                    }
                } else {
                    const float4* w4 = reinterpret_cast<const float4*>(a.norm_w);
                    for (int c = lane; c < k4; c += 32) {
                        float4 v = h4[c], g = w4[c];
                        store4(xs + (size_t)m * KP + c * 4,
                               make_float4((v.x * s) * g.x, (v.y * s) * g.y, (v.z * s) * g.z, (v.w * s) * g.w));
                    }
                }
            } else {
                for (int k = lane; k < K; k += 32) xs[(size_t)m * KP + k] = __float2bfloat16_rn(0.f);
            }
        }
    } else if (direct) {
        // this warp's columns of x, each lane the values of its place in the 16 x 16
        // operand tiles of the products: rows lane / 4 and + 8, columns 2 (lane % 4) and + 8
        const int g = lane >> 2, t2 = (lane & 3) * 2;
        const bf16* x0 = a.x + (size_t)g * a.ldx + k_begin + t2;
        const bf16* x1 = x0 + (size_t)8 * a.ldx;
#pragma unroll
        for (int s = 0; s < kDirectSteps; ++s) {
            const bool in_k = k_begin + s * 16 < k_end;
            ax[s][0] = in_k && g < M ? *reinterpret_cast<const uint32_t*>(x0 + s * 16) : 0u;
            ax[s][1] = in_k && g + 8 < M ? *reinterpret_cast<const uint32_t*>(x1 + s * 16) : 0u;
            ax[s][2] = in_k && g < M ? *reinterpret_cast<const uint32_t*>(x0 + s * 16 + 8) : 0u;
            ax[s][3] = in_k && g + 8 < M ? *reinterpret_cast<const uint32_t*>(x1 + s * 16 + 8) : 0u;
        }
    } else {
        // whole rows by bulk copies, all of them in flight at once (loads through
        // registers keep too few bytes in flight to fill the SM's path from L2 when
        // there are many rows); rows past M are zeroed here
        if (warp == 0) {
            if (lane == 0) mbar_expect_tx(&xbar, (uint32_t)M * (uint32_t)K * 2u);
            __syncwarp();
            for (int m = lane; m < M; m += 32)
                bulk_load(xs + (size_t)m * KP, a.x + (size_t)m * a.ldx, (uint32_t)K * 2u, &xbar);
        }
        const int per_row = K >> 3;  // 16-byte chunks
        for (int c = threadIdx.x; c < (MT - M) * per_row; c += WARPS * 32) {
            int m = M + c / per_row, ch = c % per_row;
            *reinterpret_cast<uint4*>(xs + (size_t)m * KP + ch * 8) = make_uint4(0, 0, 0, 0);
        }
        const bool arrived = mbar_wait(&xbar, 0);
        // the zeroed rows; and the whole CTA knows if a wait ran out (it goes on, flagged,
        // through its bounded waits: no CTA leaves with copies into its memory in flight)
        failed = __syncthreads_or(!arrived) != 0;
    }
    if (PRO == PRO_NORM) __syncthreads();
    trace_mark(a.trace, 4);
    trace_mark(a.trace, 5);

    // ---- units of eight output rows --------------------------------------------
    float best_v[ET][2];
    int best_i[ET][2];
#pragma unroll
    for (int tt = 0; tt < ET; ++tt) {
        best_v[tt][0] = best_v[tt][1] = -FLT_MAX;
        best_i[tt][0] = best_i[tt][1] = -1;
    }
    for (int i = 0;; ++i) {
        int unit = first_unit + i * unit_stride;
        if (unit >= n_units) break;
        float acc[MTILES][4];
#pragma unroll
        for (int t = 0; t < MTILES; ++t)
#pragma unroll
            for (int e = 0; e < 4; ++e) acc[t][e] = 0.f;
        const bf16* a_ptr = xs + (size_t)(lane & 15) * KP + (lane >> 4) * 8;
        // with one tile of rows, two chains of products halve the dependent latency
        float acc2[4] = {0.f, 0.f, 0.f, 0.f};
        for (int ch = 0; ch < n_chunks; ++ch) {
            const int j = i * n_chunks + ch;
            const int kb = SPLITK ? k_begin : ch * KC;
            const int ke = SPLITK ? k_end : min(K, kb + KC);
            // the whole warp leaves together if any lane's wait ran out
            if (ke > kb &&
                !__all_sync(0xffffffffu, mbar_wait(bars + (j % S), (uint32_t)(j / S) & 1u))) {
                failed = true;
                break;
            }
            // lanes 0-7: weight rows at columns k0..k0+7, lanes 8-15: k0+8..k0+15; a
            // stage of whole rows is indexed by k0, a chunk by k0 - kb
            const bf16* b_ptr = wst + (size_t)(j % S) * 8 * KCP + (size_t)(lane & 7) * KCP +
                                ((lane >> 3) & 1) * 8 - (SPLITK ? 0 : kb);
            // The fragments of the next 16 columns are asked for before the products
            // of these 16 are issued (two sets of registers), so that a product never
            // waits for the shared-memory loads just ahead of it.
            uint32_t bw[2][2], af[2][MTILES][4];
            auto load_step = [&](int buf, int k0) {
                ldmatrix_x2(bw[buf][0], bw[buf][1], b_ptr + k0);
#pragma unroll
                for (int t = 0; t < MTILES; ++t) ldmatrix_x4(af[buf][t], a_ptr + (size_t)t * 16 * KP + k0);
            };
            auto mma_step = [&](int buf) {
#pragma unroll
                for (int t = 0; t < MTILES; ++t) {
                    if (MTILES == 1 && buf == 1) mma_bf16(acc2, af[buf][t], bw[buf][0], bw[buf][1]);
                    else mma_bf16(acc[t], af[buf][t], bw[buf][0], bw[buf][1]);
                }
            };
            if (direct) {
                // x is in registers already: the weights' fragments of all steps first, then
                // the products, on two chains
                uint32_t bd[kDirectSteps][2];
#pragma unroll
                for (int s = 0; s < kDirectSteps; ++s)
                    if (kb + s * 16 < ke) ldmatrix_x2(bd[s][0], bd[s][1], b_ptr + kb + s * 16);
#pragma unroll
                for (int s = 0; s < kDirectSteps; ++s)
                    if (kb + s * 16 < ke) {
                        if (s & 1) mma_bf16(acc2, ax[s], bd[s][0], bd[s][1]);
                        else mma_bf16(acc[0], ax[s], bd[s][0], bd[s][1]);
                    }
            } else {
            int k0 = kb;
            if (k0 < ke) load_step(0, k0);
#pragma unroll 2
            for (; k0 + 32 <= ke; k0 += 32) {
                load_step(1, k0 + 16);
                mma_step(0);
                if (k0 + 32 < ke) load_step(0, k0 + 32);
                mma_step(1);
            }
            if (k0 < ke) mma_step(0);
            }
            if (!SPLITK) {
                __syncwarp();  // every lane has read this stage: it may be filled again
                if (lane == 0) issue(j + S);
            }
        }
        if (failed && !SPLITK) break;
        if (i == 0) {
            trace_mark(a.trace, 6);
            trace_mark(a.trace, 7);
        }
        if (MTILES == 1) {
#pragma unroll
            for (int e = 0; e < 4; ++e) acc[0][e] += acc2[e];
        }
        float eacc[ET][4];  // the sums that this warp finishes
        if (SPLITK) {
            // partial sums of the warps, added in warp order; warp t takes tile t
#pragma unroll
            for (int t = 0; t < MTILES; ++t)
#pragma unroll
                for (int e = 0; e < 4; ++e) red[((size_t)(warp * MTILES + t) * 4 + e) * 32 + lane] = acc[t][e];
            __syncthreads();
            if (warp >= MTILES) break;  // one unit per CTA: the other warps are done
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                float sum = red[((size_t)warp * 4 + e) * 32 + lane];
                for (int w = 1; w < WARPS; ++w) sum += red[((size_t)(w * MTILES + warp) * 4 + e) * 32 + lane];
                eacc[0][e] = sum;
            }
        } else {
#pragma unroll
            for (int tt = 0; tt < ET; ++tt)
#pragma unroll
                for (int e = 0; e < 4; ++e) eacc[tt][e] = acc[SPLITK ? 0 : tt][e];
        }

        // ---- epilogue -----------------------------------------------------------
#pragma unroll
        for (int tt = 0; tt < ET; ++tt)
            epi_finish<EPI>(a, unit, tile_of(tt) * 16, lane, eacc[tt], pre[tt], i == 0, best_v[tt], best_i[tt]);
    }
    if (failed && lane == 0 && a.status) atomicExch(a.status, 2);
    if (EPI != EPI_ARGMAX) trace_mark(a.trace, 1);

    if (EPI == EPI_ARGMAX) {
        // the four lanes of a row hold its candidates: fold them, then the warps,
        // then the CTAs; the last CTA to arrive finishes the rows.
#pragma unroll
        for (int tt = 0; tt < ET; ++tt)
#pragma unroll
            for (int hrow = 0; hrow < 2; ++hrow) {
#pragma unroll
                for (int o = 1; o < 4; o <<= 1) {
                    float ov = __shfl_xor_sync(0xffffffffu, best_v[tt][hrow], o);
                    int oi = __shfl_xor_sync(0xffffffffu, best_i[tt][hrow], o);
                    if (oi >= 0 && better(ov, oi, best_v[tt][hrow], best_i[tt][hrow])) {
                        best_v[tt][hrow] = ov;
                        best_i[tt][hrow] = oi;
                    }
                }
                // (with the warps sharing K a row has one candidate: its tile's warp's)
                if (epi_warp && (lane & 3) == 0) {
                    cta_val[SPLITK ? 0 : warp][tile_of(tt) * 16 + r_lo + hrow * 8] = best_v[tt][hrow];
                    cta_idx[SPLITK ? 0 : warp][tile_of(tt) * 16 + r_lo + hrow * 8] = best_i[tt][hrow];
                }
            }
        __syncthreads();
        for (int m = threadIdx.x; m < M; m += WARPS * 32) {
            float bv = -FLT_MAX;
            int bi = -1;
            for (int w = 0; w < (SPLITK ? 1 : WARPS); ++w) {
                if (cta_idx[w][m] >= 0 && better(cta_val[w][m], cta_idx[w][m], bv, bi)) {
                    bv = cta_val[w][m];
                    bi = cta_idx[w][m];
                }
            }
            a.best_val[(size_t)m * gridDim.x + blockIdx.x] = bv;
            a.best_idx[(size_t)m * gridDim.x + blockIdx.x] = bi;
        }
        __threadfence();
        __syncthreads();
        if (threadIdx.x == 0) is_last = atomicAdd(a.ticket, 1u) == gridDim.x - 1;
        __syncthreads();
        if (is_last) {
            __threadfence();
            for (int m = warp; m < M; m += WARPS) {
                float bv = -FLT_MAX;
                int bi = -1;
                for (int c = lane; c < (int)gridDim.x; c += 32) {
                    float v = a.best_val[(size_t)m * gridDim.x + c];
                    int ix = a.best_idx[(size_t)m * gridDim.x + c];
                    if (ix >= 0 && better(v, ix, bv, bi)) {
                        bv = v;
                        bi = ix;
                    }
                }
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) {
                    float ov = __shfl_xor_sync(0xffffffffu, bv, o);
                    int oi = __shfl_xor_sync(0xffffffffu, bi, o);
                    if (oi >= 0 && better(ov, oi, bv, bi)) {
                        bv = ov;
                        bi = oi;
                    }
                }
                if (lane == 0) {
                    int picked = bi < 0 ? 0 : bi;
                    reinterpret_cast<int*>(a.out)[m] = picked;
                    if (a.next_tokens && a.next_pos[m] >= 0) {
                        a.next_tokens[m] = picked;
                        a.next_pos[m] += 1;
                    }
                }
            }
            if (threadIdx.x == 0) *a.ticket = 0u;
        }
        trace_mark(a.trace, 1);
    }
}

struct GemvPlan {
    int mtiles, warps, stages, grid;
    int kc;  // columns of K per weight stage
    bool splitk;
    size_t smem;
};

template <int MTILES, int EPI, int PRO, int S, int WARPS, bool SPLITK>
static inline int launch_gemv_final(const GemvArgs& a, const GemvPlan& plan, bool pdl, cudaStream_t stream) {
    auto kernel = gemv_kernel<MTILES, EPI, PRO, S, WARPS, SPLITK>;
    if (plan.smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             (int)plan.smem);
        if (e != cudaSuccess) return (int)e;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(plan.grid);
    cfg.blockDim = dim3(WARPS * 32);
    cfg.dynamicSmemBytes = plan.smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 1 : 0;
    cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, a);
    return e == cudaSuccess ? NNIS_OK : (int)e;
}

template <int MTILES, int EPI, int PRO>
static inline int launch_gemv_shape(const GemvArgs& a, const GemvPlan& p, bool pdl, cudaStream_t stream) {
    if (p.splitk) return launch_gemv_final<MTILES, EPI, PRO, 1, 8, true>(a, p, pdl, stream);
    if (p.warps == 8)
        return p.stages == 2 ? launch_gemv_final<MTILES, EPI, PRO, 2, 8, false>(a, p, pdl, stream)
                             : launch_gemv_final<MTILES, EPI, PRO, 1, 8, false>(a, p, pdl, stream);
    return p.stages == 2 ? launch_gemv_final<MTILES, EPI, PRO, 2, 4, false>(a, p, pdl, stream)
                         : launch_gemv_final<MTILES, EPI, PRO, 1, 4, false>(a, p, pdl, stream);
}

template <int MTILES>
int launch_gemv_epi(const GemvArgs& a, int epi, int pro, const GemvPlan& p, bool pdl,
                           cudaStream_t stream) {
#define NNIS_GEMV(EPI, PRO) return launch_gemv_shape<MTILES, EPI, PRO>(a, p, pdl, stream)
    // the pairs of prologue and epilogue that the decode step uses
    if (epi == EPI_QKV && pro == PRO_NORM) NNIS_GEMV(EPI_QKV, PRO_NORM);
    if (epi == EPI_QKV && pro == PRO_PLAIN) NNIS_GEMV(EPI_QKV, PRO_PLAIN);
    if (epi == EPI_GATED && pro == PRO_NORM) NNIS_GEMV(EPI_GATED, PRO_NORM);
    if (epi == EPI_GATED && pro == PRO_PLAIN) NNIS_GEMV(EPI_GATED, PRO_PLAIN);
    if (epi == EPI_ADD_F32 && pro == PRO_PLAIN) NNIS_GEMV(EPI_ADD_F32, PRO_PLAIN);
    if (epi == EPI_STORE && pro == PRO_PLAIN) NNIS_GEMV(EPI_STORE, PRO_PLAIN);
    if (epi == EPI_STORE_F32 && pro == PRO_PLAIN) NNIS_GEMV(EPI_STORE_F32, PRO_PLAIN);
    if (epi == EPI_STORE_F32 && pro == PRO_NORM) NNIS_GEMV(EPI_STORE_F32, PRO_NORM);
    if (epi == EPI_ARGMAX && pro == PRO_NORM) NNIS_GEMV(EPI_ARGMAX, PRO_NORM);
    if (epi == EPI_ARGMAX && pro == PRO_PLAIN) NNIS_GEMV(EPI_ARGMAX, PRO_PLAIN);
#undef NNIS_GEMV
    return NNIS_ERR_UNSUPPORTED;
}

}  // namespace nnis
