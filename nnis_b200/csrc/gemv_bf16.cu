// Projections of a decode step in bfloat16: y[M, N] = x[M, K] . W[N, K]^T with
// at most 16 rows of x.  The step is bound by the bytes of W and by latency, so
//
//  * W is brought into shared memory by bulk asynchronous copies (one per
//    weight row, completing on an mbarrier), issued before anything else in the
//    kernel - before the wait of programmatic dependent launch, hence while the
//    kernel before it still runs - and double-buffered per warp;
//  * what surrounds the product is fused so that no activation makes a round
//    trip through its own kernel:
//      prologue  NORM:  x = bf16(rmsnorm(hidden_f32[rows]) * w_norm);
//                MERGE: x = bf16(attention output) merged from the split-KV
//                       partial records of the decode attention kernel;
//      epilogue  STORE (bfloat16), STORE_F32, ADD_F32 (into the residual stream),
//                GATED:  out[m, i] = bf16(silu(y[m, i]) * y[m, I + i]),
//                QKV:    bias, round, rotate-half RoPE of q and k heads at each
//                        row's position, q to a packed buffer, k and v into the
//                        paged cache,
//                ARGMAX: the index of the largest y per row (ties to the lower
//                        index), optionally the float32 logits too, and the move
//                        of the decode state to the next token.
//
// A warp owns four output rows at a time (a "unit"); lanes split K in chunks of
// eight.  Sums are float32 fmaf chains, reduced across the warp by a butterfly.
// NNIS's one-token projection: crates/nnis-kernels/src/gemv.rs:45-61; its fused
// gate/up/SiLU kernel: crates/nnis-model/src/fused_swiglu.rs:14-27; its greedy
// pick: crates/nnis-kernels/src/top_k.rs:57-70.
#include <float.h>

#include "async_copy.cuh"
#include "common.cuh"

namespace nnis {

enum { EPI_STORE = 0, EPI_STORE_F32 = 1, EPI_ADD_F32 = 2, EPI_GATED = 3, EPI_QKV = 4, EPI_ARGMAX = 5 };
enum { PRO_PLAIN = 0, PRO_NORM = 1, PRO_MERGE = 2 };

struct GemvArgs {
    const bf16* x;          // [M, K] (plain prologue)
    const float* hidden;    // [*, K] float32 residual stream (norm prologue)
    const int* rows;        // optional row of `hidden` per x row
    const float* norm_w;    // [K]
    float eps;
    const float* partial;   // merge prologue: [M * nq, splits, d + 2]
    int splits;
    const bf16* w;          // [N, K]
    const float* bias;      // [N] or null
    void* out;              // see epilogues
    int M, N, K;
    int* status;            // set non-zero when a bounded wait runs out
    // QKV epilogue (nq, d also describe the merge prologue)
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
};

__device__ __forceinline__ void unpack8f(const uint4& raw, float* f) {
    f[0] = __uint_as_float(raw.x << 16);
    f[1] = __uint_as_float(raw.x & 0xffff0000u);
    f[2] = __uint_as_float(raw.y << 16);
    f[3] = __uint_as_float(raw.y & 0xffff0000u);
    f[4] = __uint_as_float(raw.z << 16);
    f[5] = __uint_as_float(raw.z & 0xffff0000u);
    f[6] = __uint_as_float(raw.w << 16);
    f[7] = __uint_as_float(raw.w & 0xffff0000u);
}

__device__ __forceinline__ float round_bf16(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }

// value number `idx` of a register array, without dynamic indexing
template <int COUNT>
__device__ __forceinline__ float pick(const float* v, int idx) {
    float r = 0.f;
#pragma unroll
    for (int i = 0; i < COUNT; ++i) r = (idx == i) ? v[i] : r;
    return r;
}

__device__ __forceinline__ bool better(float v, int i, float bv, int bi) {
    return bi < 0 || v > bv || (v == bv && i < bi);
}

constexpr int kGemvWarps = 8;

template <int EPI>
__device__ __forceinline__ void unit_rows(const GemvArgs& a, int unit, int& r0, int& r2) {
    if (EPI == EPI_GATED) {
        r0 = unit * 2;
        r2 = (a.N >> 1) + unit * 2;
    } else if (EPI == EPI_QKV) {
        int per_head = a.d >> 2;
        int head = unit / per_head, jj = (unit - head * per_head) * 2;
        r0 = head * a.d + jj;
        r2 = r0 + (a.d >> 1);
    } else {
        r0 = unit * 4;
        r2 = r0 + 2;
    }
}

template <int MT, int EPI, int PRO, int S>
__global__ void __launch_bounds__(kGemvWarps * 32)
gemv_kernel(GemvArgs a) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int K = a.K, M = a.M;
    bf16* xs = reinterpret_cast<bf16*>(smem_raw);                                    // [MT, K]
    bf16* wst = xs + (size_t)MT * K + (size_t)warp * S * 4 * K;                      // [S, 4, K]
    uint64_t* bars = reinterpret_cast<uint64_t*>(xs + (size_t)(MT + kGemvWarps * S * 4) * K) + warp * S;
    __shared__ float cta_val[kGemvWarps][MT];
    __shared__ int cta_idx[kGemvWarps][MT];
    __shared__ bool is_last;

    const int n_units = a.N >> 2;
    const int unit_stride = gridDim.x * kGemvWarps;
    const int first_unit = blockIdx.x * kGemvWarps + warp;
    const uint32_t row_bytes = (uint32_t)K * 2u;

    auto issue = [&](int i) {  // lane 0 only
        int unit = first_unit + i * unit_stride;
        if (unit >= n_units) return;
        int r0, r2;
        unit_rows<EPI>(a, unit, r0, r2);
        uint64_t* bar = bars + (i % S);
        bf16* dst = wst + (size_t)(i % S) * 4 * K;
        mbar_expect_tx(bar, 4u * row_bytes);
        bulk_load(dst, a.w + (size_t)r0 * K, row_bytes, bar);
        bulk_load(dst + K, a.w + (size_t)(r0 + 1) * K, row_bytes, bar);
        bulk_load(dst + 2 * (size_t)K, a.w + (size_t)r2 * K, row_bytes, bar);
        bulk_load(dst + 3 * (size_t)K, a.w + (size_t)(r2 + 1) * K, row_bytes, bar);
    };

    // ---- weights first: they depend on no earlier kernel ---------------------
    if (lane == 0) {
#pragma unroll
        for (int s = 0; s < S; ++s) mbar_init(bars + s, 1);
        mbar_fence_init();
#pragma unroll
        for (int s = 0; s < S; ++s) issue(s);
    }
    // what does not depend on earlier kernels: the norm weights of this lane's columns
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
    // Dependents are released only after this kernel's own wait: a kernel that
    // starts early may then rely on everything before its immediate predecessor
    // (the decode attention kernel reads old cache pages before its wait).
    pdl_wait();
    pdl_launch_dependents();

    // operands of the first unit's epilogue, asked for now and used after the products
    const int lane_m = (EPI == EPI_QKV) ? (lane >> 1) : (lane >> 2);
    int pre_pos = -1;
    if (EPI == EPI_QKV && lane_m < M) pre_pos = a.token_pos[lane_m];

    // ---- x into shared memory ------------------------------------------------
    if (PRO == PRO_NORM) {
        const bool in_regs = k4 <= 32 * NW;
        for (int m = warp; m < MT; m += kGemvWarps) {
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
                    for (int k = lane; k < K; k += 32) ss = fmaf(h[k], h[k], ss);
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
                            store4(xs + (size_t)m * K + c * 4, r);
                        }
                    }
                } else {
                    for (int k = lane; k < K; k += 32)
                        xs[(size_t)m * K + k] = __float2bfloat16_rn((h[k] * s) * a.norm_w[k]);
                }
            } else {
                for (int k = lane; k < K; k += 32) xs[(size_t)m * K + k] = __float2bfloat16_rn(0.f);
            }
        }
    } else if (PRO == PRO_MERGE) {
        // one warp per (row, head): weights of the splits, then the weighted sum
        const int d = a.d, nq = a.nq, sp = a.splits;
        for (int p = warp; p < MT * nq; p += kGemvWarps) {
            int m = p / nq, hq = p - m * nq;
            bf16* dst = xs + (size_t)m * K + (size_t)hq * d;
            if (m >= M) {
                for (int i = lane; i < d; i += 32) dst[i] = __float2bfloat16_rn(0.f);
                continue;
            }
            const float* rec = a.partial + ((size_t)m * nq + hq) * sp * (size_t)(d + 2);
            float m0 = -FLT_MAX, l0 = 0.f, m1 = -FLT_MAX, l1 = 0.f;
            if (lane < sp) {
                m0 = rec[(size_t)lane * (d + 2)];
                l0 = rec[(size_t)lane * (d + 2) + 1];
            }
            if (lane + 32 < sp) {
                m1 = rec[(size_t)(lane + 32) * (d + 2)];
                l1 = rec[(size_t)(lane + 32) * (d + 2) + 1];
            }
            float mx = warp_max(fmaxf(l0 > 0.f ? m0 : -FLT_MAX, l1 > 0.f ? m1 : -FLT_MAX));
            float w0 = l0 > 0.f ? __expf(m0 - mx) : 0.f;
            float w1 = l1 > 0.f ? __expf(m1 - mx) : 0.f;
            float total = warp_sum(l0 * w0 + l1 * w1);
            float inv = total > 0.f ? 1.0f / total : 0.f;
            for (int i0 = 0; i0 < d; i0 += 32) {
                int i = i0 + lane;
                float o = 0.f;
                for (int s = 0; s < sp; ++s) {
                    float ws = __shfl_sync(0xffffffffu, s < 32 ? w0 : w1, s & 31);
                    if (i < d) o = fmaf(ws, rec[(size_t)s * (d + 2) + 2 + i], o);
                }
                if (i < d) dst[i] = __float2bfloat16_rn(o * inv);
            }
        }
    } else {
        const int chunks = MT * K / 8;
        for (int c = threadIdx.x; c < chunks; c += kGemvWarps * 32) {
            int m = (c * 8) / K;
            uint4 v = make_uint4(0, 0, 0, 0);
            if (m < M) v = *reinterpret_cast<const uint4*>(a.x + (size_t)c * 8);
            *reinterpret_cast<uint4*>(xs + (size_t)c * 8) = v;
        }
    }
    __syncthreads();

    // ---- units of four output rows ---------------------------------------------
    const int half = a.d >> 1;
    const int inter = a.N >> 1;
    float pre_c = 1.f, pre_s = 0.f, pre_old0 = 0.f, pre_old1 = 0.f;
    int pre_page = 0;
    if (first_unit < n_units) {
        int r0, r2;
        unit_rows<EPI>(a, first_unit, r0, r2);
        if (EPI == EPI_QKV && pre_pos >= 0) {
            int head = r0 / a.d, j = r0 - head * a.d + (lane & 1);
            if (a.sin_t && head < a.nq + a.nkv) {
                pre_c = a.cos_t[(size_t)pre_pos * half + j];
                pre_s = a.sin_t[(size_t)pre_pos * half + j];
            }
            if (head >= a.nq)
                pre_page = a.page_table[(size_t)a.token_seq[lane_m] * a.table_cols + pre_pos / a.page_size];
        }
        if (EPI == EPI_ADD_F32) {
            int r = lane & 3;
            int n = (r < 2 ? r0 + r : r2 + r - 2);
            if (lane_m < M) pre_old0 = reinterpret_cast<const float*>(a.out)[(size_t)lane_m * a.N + n];
            if (MT * 4 > 32 && lane_m + 8 < M)
                pre_old1 = reinterpret_cast<const float*>(a.out)[(size_t)(lane_m + 8) * a.N + n];
        }
    }
    constexpr int SLOTS = (MT * 4 + 31) / 32;
    float best_v[SLOTS];
    int best_i[SLOTS];
#pragma unroll
    for (int t = 0; t < SLOTS; ++t) {
        best_v[t] = -FLT_MAX;
        best_i[t] = -1;
    }
    bool failed = false;
    for (int i = 0;; ++i) {
        int unit = first_unit + i * unit_stride;
        if (unit >= n_units) break;
        int r0, r2;
        unit_rows<EPI>(a, unit, r0, r2);
        // the whole warp leaves together if any lane's wait ran out
        if (!__all_sync(0xffffffffu, mbar_wait(bars + (i % S), (uint32_t)(i / S) & 1u))) {
            failed = true;
            break;
        }
        const bf16* wbuf = wst + (size_t)(i % S) * 4 * K;
        float acc[MT * 4];
#pragma unroll
        for (int j = 0; j < MT * 4; ++j) acc[j] = 0.f;
        for (int k = lane * 8; k < K; k += 256) {
            float f0[8], f1[8], f2[8], f3[8];
            unpack8f(*reinterpret_cast<const uint4*>(wbuf + k), f0);
            unpack8f(*reinterpret_cast<const uint4*>(wbuf + K + k), f1);
            unpack8f(*reinterpret_cast<const uint4*>(wbuf + 2 * (size_t)K + k), f2);
            unpack8f(*reinterpret_cast<const uint4*>(wbuf + 3 * (size_t)K + k), f3);
#pragma unroll
            for (int m = 0; m < MT; ++m) {
                float xf[8];
                unpack8f(*reinterpret_cast<const uint4*>(xs + (size_t)m * K + k), xf);
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                    acc[m * 4 + 0] = fmaf(xf[e], f0[e], acc[m * 4 + 0]);
                    acc[m * 4 + 1] = fmaf(xf[e], f1[e], acc[m * 4 + 1]);
                    acc[m * 4 + 2] = fmaf(xf[e], f2[e], acc[m * 4 + 2]);
                    acc[m * 4 + 3] = fmaf(xf[e], f3[e], acc[m * 4 + 3]);
                }
            }
        }
        __syncwarp();  // every lane has read this stage: it may be filled again
        if (lane == 0) issue(i + S);
#pragma unroll
        for (int j = 0; j < MT * 4; ++j) acc[j] = warp_sum(acc[j]);

        // ---- epilogue: lane j finishes value j (two passes when MT = 16) ---------
#pragma unroll
        for (int pass = 0; pass < SLOTS; ++pass) {
            if (EPI == EPI_GATED || EPI == EPI_QKV) {
                // pairs: (m, p) with partner row r2 + p; 2 * MT pairs
                int idx = pass * 32 + lane;
                int m = idx >> 1, p = idx & 1;
                if (idx < MT * 2 && m < M) {
                    float va = pick<MT * 4>(acc, m * 4 + p);
                    float vb = pick<MT * 4>(acc, m * 4 + 2 + p);
                    if (a.bias) {
                        va += a.bias[r0 + p];
                        vb += a.bias[r2 + p];
                    }
                    if (EPI == EPI_GATED) {
                        bf16* out = reinterpret_cast<bf16*>(a.out);
                        out[(size_t)m * inter + unit * 2 + p] =
                            __float2bfloat16_rn((va / (1.0f + expf(-va))) * vb);
                    } else {
                        const bool first = (i == 0);
                        int pos = first ? pre_pos : a.token_pos[m];
                        if (pos >= 0) {
                            int head = r0 / a.d, j = r0 - head * a.d + p;
                            va = round_bf16(va);
                            vb = round_bf16(vb);
                            bool is_v = head >= a.nq + a.nkv;
                            if (a.sin_t && !is_v) {
                                float c = first ? pre_c : a.cos_t[(size_t)pos * half + j];
                                float s = first ? pre_s : a.sin_t[(size_t)pos * half + j];
                                float ra = va * c - vb * s, rb = vb * c + va * s;
                                va = ra;
                                vb = rb;
                            }
                            bf16 ta = __float2bfloat16_rn(va), tb = __float2bfloat16_rn(vb);
                            if (head < a.nq) {
                                bf16* out = reinterpret_cast<bf16*>(a.out) +
                                            ((size_t)m * a.nq + head) * a.d;
                                out[j] = ta;
                                out[j + half] = tb;
                            } else {
                                int hk = is_v ? head - a.nq - a.nkv : head - a.nq;
                                bf16* cache = is_v ? a.v_cache : a.k_cache;
                                int page = first ? pre_page
                                                 : a.page_table[(size_t)a.token_seq[m] * a.table_cols +
                                                                pos / a.page_size];
                                size_t dst = ((size_t)(page * a.nkv + hk) * a.page_size +
                                              (pos % a.page_size)) * a.d;
                                cache[dst + j] = ta;
                                cache[dst + j + half] = tb;
                            }
                        }
                    }
                }
            } else {
                int idx = pass * 32 + lane;
                int m = idx >> 2, r = idx & 3;
                if (idx < MT * 4 && m < M) {
                    int n = (r < 2 ? r0 + r : r2 + r - 2);
                    float v = pick<MT * 4>(acc, idx) + (a.bias ? a.bias[n] : 0.f);
                    size_t o = (size_t)m * a.N + n;
                    if (EPI == EPI_STORE) reinterpret_cast<bf16*>(a.out)[o] = __float2bfloat16_rn(v);
                    else if (EPI == EPI_STORE_F32) reinterpret_cast<float*>(a.out)[o] = v;
                    else if (EPI == EPI_ADD_F32) {
                        float old = (i == 0) ? (pass == 0 ? pre_old0 : pre_old1)
                                             : reinterpret_cast<const float*>(a.out)[o];
                        reinterpret_cast<float*>(a.out)[o] = old + v;
                    }
                    else {
                        if (a.logits) a.logits[o] = v;
                        if (better(v, n, best_v[pass], best_i[pass])) {
                            best_v[pass] = v;
                            best_i[pass] = n;
                        }
                    }
                }
            }
        }
    }
    if (failed && lane == 0 && a.status) atomicExch(a.status, 2);

    if (EPI == EPI_ARGMAX) {
        // lanes 4m .. 4m+3 (of pass p) hold row m's candidates: fold them, then the
        // warps, then the CTAs; the last CTA to arrive finishes the rows.
#pragma unroll
        for (int pass = 0; pass < SLOTS; ++pass) {
#pragma unroll
            for (int o = 1; o < 4; o <<= 1) {
                float ov = __shfl_xor_sync(0xffffffffu, best_v[pass], o);
                int oi = __shfl_xor_sync(0xffffffffu, best_i[pass], o);
                if (oi >= 0 && better(ov, oi, best_v[pass], best_i[pass])) {
                    best_v[pass] = ov;
                    best_i[pass] = oi;
                }
            }
            int m = (pass * 32 + lane) >> 2;
            if ((lane & 3) == 0 && m < MT) {
                cta_val[warp][m] = best_v[pass];
                cta_idx[warp][m] = best_i[pass];
            }
        }
        __syncthreads();
        if (threadIdx.x < MT && threadIdx.x < M) {
            int m = threadIdx.x;
            float bv = -FLT_MAX;
            int bi = -1;
            for (int w = 0; w < kGemvWarps; ++w) {
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
            for (int m = warp; m < M; m += kGemvWarps) {
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
    }
}

template <int MT, int EPI, int PRO, int S>
static int launch_gemv_final(const GemvArgs& a, int grid, size_t smem, bool pdl, cudaStream_t stream) {
    auto kernel = gemv_kernel<MT, EPI, PRO, S>;
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             (int)smem);
        if (e != cudaSuccess) return (int)e;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(kGemvWarps * 32);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 1 : 0;
    cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, a);
    return e == cudaSuccess ? NNIS_OK : (int)e;
}

template <int MT, int EPI, int PRO>
static int launch_gemv_stages(const GemvArgs& a, int stages, int grid, size_t smem, bool pdl,
                              cudaStream_t stream) {
    if (stages == 2) return launch_gemv_final<MT, EPI, PRO, 2>(a, grid, smem, pdl, stream);
    return launch_gemv_final<MT, EPI, PRO, 1>(a, grid, smem, pdl, stream);
}

template <int MT>
static int launch_gemv_epi(const GemvArgs& a, int epi, int pro, int stages, int grid, size_t smem,
                           bool pdl, cudaStream_t stream) {
#define NNIS_GEMV(EPI, PRO) return launch_gemv_stages<MT, EPI, PRO>(a, stages, grid, smem, pdl, stream)
    // the pairs of prologue and epilogue that the decode step uses
    if (epi == EPI_QKV && pro == PRO_NORM) NNIS_GEMV(EPI_QKV, PRO_NORM);
    if (epi == EPI_QKV && pro == PRO_PLAIN) NNIS_GEMV(EPI_QKV, PRO_PLAIN);
    if (epi == EPI_GATED && pro == PRO_NORM) NNIS_GEMV(EPI_GATED, PRO_NORM);
    if (epi == EPI_GATED && pro == PRO_PLAIN) NNIS_GEMV(EPI_GATED, PRO_PLAIN);
    if (epi == EPI_ADD_F32 && pro == PRO_PLAIN) NNIS_GEMV(EPI_ADD_F32, PRO_PLAIN);
    if (epi == EPI_ADD_F32 && pro == PRO_MERGE) NNIS_GEMV(EPI_ADD_F32, PRO_MERGE);
    if (epi == EPI_STORE && pro == PRO_PLAIN) NNIS_GEMV(EPI_STORE, PRO_PLAIN);
    if (epi == EPI_STORE_F32 && pro == PRO_PLAIN) NNIS_GEMV(EPI_STORE_F32, PRO_PLAIN);
    if (epi == EPI_STORE_F32 && pro == PRO_NORM) NNIS_GEMV(EPI_STORE_F32, PRO_NORM);
    if (epi == EPI_ARGMAX && pro == PRO_NORM) NNIS_GEMV(EPI_ARGMAX, PRO_NORM);
    if (epi == EPI_ARGMAX && pro == PRO_PLAIN) NNIS_GEMV(EPI_ARGMAX, PRO_PLAIN);
#undef NNIS_GEMV
    return NNIS_ERR_UNSUPPORTED;
}

}  // namespace nnis

// How many CTAs a launch with these sizes has: the ARGMAX scratch is
// [M, this many] values and indices.
NNIS_API int nnis_gemv_grid(int M, int N, int K, int sm_count) {
    int units = N / 4;
    int grid = (units + nnis::kGemvWarps - 1) / nnis::kGemvWarps;
    int cap = (sm_count > 0 ? sm_count : 148) * 2;
    return grid > cap ? cap : grid;
}

// Refuses (NNIS_ERR_UNSUPPORTED) what it does not take: M > 16, K not a multiple
// of 8, N not a multiple of 4, operands too large for shared memory; the caller
// then takes the general kernels.  Scratch: the merge prologue reads `partial`
// (written by the decode attention kernel); the ARGMAX epilogue uses `best_val`,
// `best_idx` ([M, nnis_gemv_grid()] each) and `ticket` (one zeroed counter).
NNIS_API int nnis_gemv_bf16(const void* x, const float* hidden, const int* rows, const float* norm_w,
                            float eps, const float* partial, int splits, const void* w,
                            const float* bias, void* out, int M, int N, int K, int epilogue,
                            const int* token_pos, const int* token_seq, const int* page_table,
                            int table_cols, const float* cos_t, const float* sin_t, void* k_cache,
                            void* v_cache, int nq, int nkv, int d, int page_size, float* logits,
                            float* best_val, int* best_idx, unsigned* ticket, int* next_tokens,
                            int* next_pos, int* status, int sm_count, int pdl, cudaStream_t stream) {
    using namespace nnis;
    if (M <= 0 || N <= 0 || K <= 0 || !w || !out) return NNIS_ERR_ARGUMENT;
    if (M > 16 || K % 8 || N % 4) return NNIS_ERR_UNSUPPORTED;
    int pro = hidden ? PRO_NORM : (partial ? PRO_MERGE : PRO_PLAIN);
    if (pro == PRO_PLAIN && !x) return NNIS_ERR_ARGUMENT;
    if (pro == PRO_NORM && (!norm_w || !(eps > 0.f))) return NNIS_ERR_ARGUMENT;
    if (pro == PRO_MERGE && (splits <= 0 || splits > 64 || nq <= 0 || d <= 0 || nq * d != K))
        return NNIS_ERR_ARGUMENT;
    if (((uintptr_t)w | (uintptr_t)x) % 16) return NNIS_ERR_ALIGNMENT;
    if (epilogue == EPI_GATED && N % 8) return NNIS_ERR_UNSUPPORTED;
    if (epilogue == EPI_QKV) {
        if (!token_pos || d <= 0 || d % 4 || N != (nq + 2 * nkv) * d) return NNIS_ERR_ARGUMENT;
        if (nkv > 0 && (!token_seq || !page_table || !k_cache || !v_cache || page_size <= 0))
            return NNIS_ERR_ARGUMENT;
    }
    if (epilogue == EPI_ARGMAX && (!best_val || !best_idx || !ticket)) return NNIS_ERR_ARGUMENT;
    if (epilogue == EPI_ARGMAX && next_tokens && !next_pos) return NNIS_ERR_ARGUMENT;
    int mt = M <= 1 ? 1 : M <= 2 ? 2 : M <= 4 ? 4 : M <= 8 ? 8 : 16;
    int grid = nnis_gemv_grid(M, N, K, sm_count);
    int units = N / 4;
    // a second stage only pays when a warp has more than one unit
    int stages = units > grid * kGemvWarps ? 2 : 1;
    auto bytes = [&](int s) {
        return ((size_t)mt + (size_t)kGemvWarps * s * 4) * K * sizeof(bf16) + kGemvWarps * s * 8;
    };
    if (stages == 2 && bytes(2) > 100 * 1024) stages = 1;
    size_t smem = bytes(stages);
    if (smem > 200 * 1024) return NNIS_ERR_UNSUPPORTED;
    GemvArgs a;
    a.x = (const bf16*)x; a.hidden = hidden; a.rows = rows; a.norm_w = norm_w; a.eps = eps;
    a.partial = partial; a.splits = splits;
    a.w = (const bf16*)w; a.bias = bias; a.out = out; a.M = M; a.N = N; a.K = K; a.status = status;
    a.token_pos = token_pos; a.token_seq = token_seq; a.page_table = page_table;
    a.table_cols = table_cols; a.cos_t = cos_t; a.sin_t = sin_t; a.k_cache = (bf16*)k_cache;
    a.v_cache = (bf16*)v_cache; a.nq = nq; a.nkv = nkv; a.d = d > 0 ? d : 4; a.page_size = page_size;
    a.logits = logits; a.best_val = best_val; a.best_idx = best_idx; a.ticket = ticket;
    a.next_tokens = next_tokens; a.next_pos = next_pos;
    switch (mt) {
        case 1: return launch_gemv_epi<1>(a, epilogue, pro, stages, grid, smem, pdl != 0, stream);
        case 2: return launch_gemv_epi<2>(a, epilogue, pro, stages, grid, smem, pdl != 0, stream);
        case 4: return launch_gemv_epi<4>(a, epilogue, pro, stages, grid, smem, pdl != 0, stream);
        case 8: return launch_gemv_epi<8>(a, epilogue, pro, stages, grid, smem, pdl != 0, stream);
        default: return launch_gemv_epi<16>(a, epilogue, pro, stages, grid, smem, pdl != 0, stream);
    }
}
