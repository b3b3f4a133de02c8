// Decode projections with few output features (a model's width, not its vocabulary):
// y[M, N] = x[M, K] . W[N, K]^T, the rows of x cut into tiles of 16.
//
// The kernel of gemv_kernel.cuh gives a CTA all rows of x for eight output features.
// With many rows it is bound by x: every CTA fetches all of it after the wait of
// programmatic dependent launch, M / 8 times the bytes of W in total, all CTAs asking L2
// for the same lines at once.  Here
//
//  * CTA (bx, by) owns NU units of eight output features (bx) for ONE tile of 16 rows
//    (by).  Its weights (NU * 8 rows of W, whole) come by bulk copies issued before the
//    wait, so W is read once per tile of rows from L2, under the kernel before this one;
//    after the wait a CTA needs only its 16 rows of x.
//  * The eight warps share K.  With x as it is (no norm) a warp takes its columns of the
//    16 rows from global memory straight into the registers of its products, eight bytes
//    a load: a lane's four consecutive columns stand for the two pairs of columns (2t,
//    2t+1 and 2t+8, 2t+9) that the tensor-core tile wants from it, and the weights are
//    read from shared memory in the same order, so the sum over K is the same sum.  With
//    the norm in front the warps normalise the rows into shared memory first: a warp to a
//    row with at most eight rows, else half a warp to a row, two rows at a time.
//  * The partial sums meet in shared memory, in the place of the weights; warp u adds
//    those of unit u in warp order (deterministic) and runs its epilogue (the ones of
//    gemv_kernel.cuh, except ARGMAX).
//  * A norm between two of these products can be shared out between them (PRO_SCALED).
//    The projection before it, whose epilogue holds the new residual values in registers,
//    also writes them times the norm's weights, in bfloat16, and each unit's share of the
//    rows' sums of squares; the projection after it takes that x as it is and multiplies
//    its float32 sums by the rows' scales, which it adds up from the shares while its
//    products run: y = scale(row) . (W . (h * w)) is the same sum as W . (h * scale * w)
//    up to the place of one rounding.  It saves the second kernel the float32 rows, the
//    pass through shared memory and a barrier between its wait and its products.
//  * A decode step is a chain of short kernels, each of which starts while the one before
//    it still runs (to fetch its weights) and must find room beside it: registers and
//    shared memory per CTA are held down on purpose (__maxnreg__; with at most eight rows
//    the second half of the tile of x is one row of zeros), so that this kernel's CTAs
//    and those of the decode attention kernel (three to an SM) are resident together.
#include <stdlib.h>

#include "gemv_kernel.cuh"

namespace nnis {

constexpr int kRowtileWarps = 8;
// 16-column steps of one warp of x in registers: K <= 768, or K <= 1,536 (LONGK)
__host__ __device__ constexpr int rowtile_direct_steps(bool longk) { return longk ? 12 : 6; }

// Registers per thread (see above), and the CTAs that fit an SM by them.
__host__ __device__ constexpr int rowtile_registers(int epi, int pro, bool longk) {
    // (the QKV epilogue holds positions, pages and angles: at 80 registers it spills)
    // (x as the kernel before weighted it: as few registers as with the norm, while K is short)
    return pro == PRO_NORM || (pro == PRO_SCALED && !longk) ? (epi == EPI_QKV ? 88 : 80) : longk ? 128 : 104;
}
__host__ __device__ constexpr int rowtile_ctas_per_sm(int epi, int pro, bool longk) {
    return 65536 / (kRowtileWarps * 32 * rowtile_registers(epi, pro, longk));
}

// Rows of the normalised x in shared memory: a tile, or eight rows and one of zeros.
__host__ __device__ constexpr int rowtile_x_rows(int M) { return M <= 8 ? 9 : 16; }

// Elements between rows of W in shared memory.  Read by ldmatrix (norm prologue:
// rows of 16 bytes, eight of them a phase) the stride must be 16 bytes off a multiple
// of 128; read by 8-byte loads, lane (g, t) at row g and 8 t bytes (half a warp a
// phase: four rows), 32 bytes off.
__host__ __device__ constexpr int rowtile_w_stride(int K, int pro) {
    return pro == PRO_NORM ? K + 8 : K + ((16 - K % 64) + 64) % 64;
}

template <int EPI, int PRO, int NU, bool LONGK>
__global__ void __maxnreg__(rowtile_registers(EPI, PRO, LONGK))
gemv_rowtile_kernel(GemvArgs a) {
    constexpr int WARPS = kRowtileWarps;
    constexpr bool kDirect = PRO != PRO_NORM;
    constexpr bool kScaled = PRO == PRO_SCALED;
    constexpr int kSteps = kDirect ? rowtile_direct_steps(LONGK) : 1;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    __shared__ __align__(8) uint64_t wbar;
    __shared__ float row_scale[16];  // PRO_SCALED: 1 / sqrt(mean of squares + eps) of the tile's rows
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    trace_mark(a.trace, 0);
    if (a.release_early) pdl_launch_dependents();
    const int K = a.K, KP = K + 8, KPW = rowtile_w_stride(K, PRO);
    const int row0 = blockIdx.y * 16;
    const int n_units = a.N >> 3;
    const int unit0 = blockIdx.x * NU;
    const int units_here = min(NU, n_units - unit0);
    bf16* ws = reinterpret_cast<bf16*>(smem_raw);                       // [NU * 8, KPW]
    const int xrows = rowtile_x_rows(a.M);
    bf16* xs = ws + (size_t)NU * 8 * KPW;                               // [xrows, KP], norm prologue only
    float* stash = reinterpret_cast<float*>(xs + (kDirect ? 0 : (size_t)xrows * KP));  // [K], more than 8 rows only
    // the partial sums take the place of the weights once every warp is through with them
    float* red = reinterpret_cast<float*>(smem_raw);                    // [WARPS, NU, 4, 32]

    // this warp's columns of K
    const int steps = K >> 4;
    const int steps_per_warp = (steps + WARPS - 1) / WARPS;
    const int k_begin = min(steps, warp * steps_per_warp) * 16;
    const int k_end = min(steps, (warp + 1) * steps_per_warp) * 16;

    // ---- weights first: they depend on no earlier kernel ---------------------
    if (warp == 0) {
        if (lane == 0) {
            mbar_init(&wbar, 1);
            mbar_fence_init();
            mbar_expect_tx(&wbar, (uint32_t)units_here * 8u * (uint32_t)K * 2u);
        }
        __syncwarp();
        for (int r = lane; r < units_here * 8; r += 32)
            bulk_load(ws + (size_t)r * KPW, a.w + (size_t)unit_row<EPI>(a, unit0 + (r >> 3), r & 7) * a.ldw,
                      (uint32_t)K * 2u, &wbar);
    }
    // ... the norm weights and what the epilogue needs.  This preamble has to fit under
    // the tail of the kernel before, so its loads are asked for before the first of them
    // is used.  With at most eight rows a warp normalises one row and keeps its share of
    // the norm weights in registers; with more they go to shared memory.
    constexpr int NW = 12;  // float4 of a row per lane of a half warp kept in registers: covers K <= 768
    constexpr int NWF = 6;  // ... per lane of a whole warp
    constexpr int kStashPer = 2;  // float4 per thread: the stash covers K <= 2,048
    const int k4 = K >> 2;
    const bool few = a.M <= 8;
    const bool stashed = PRO == PRO_NORM && !few && k4 <= kStashPer * WARPS * 32;
    float4 sv[kStashPer], nw[NWF];
    if (PRO == PRO_NORM && few) {
#pragma unroll
        for (int j = 0; j < NWF; ++j) {
            int c = lane + 32 * j;
            nw[j] = c < k4 ? reinterpret_cast<const float4*>(a.norm_w)[c] : make_float4(0.f, 0.f, 0.f, 0.f);
        }
    }
    if (stashed) {
#pragma unroll
        for (int j = 0; j < kStashPer; ++j) {
            int c = threadIdx.x + j * WARPS * 32;
            sv[j] = c < k4 ? reinterpret_cast<const float4*>(a.norm_w)[c] : make_float4(0.f, 0.f, 0.f, 0.f);
        }
    }
    const bool epi_warp = warp < units_here;
    EpiTile pre;
    if (epi_warp) epi_preload<EPI>(a, unit0 + warp, row0, lane, false, pre);
    if (stashed) {
#pragma unroll
        for (int j = 0; j < kStashPer; ++j) {
            int c = threadIdx.x + j * WARPS * 32;
            if (c < k4) reinterpret_cast<float4*>(stash)[c] = sv[j];
        }
    }
    const float4* w4 = stashed ? reinterpret_cast<const float4*>(stash) : reinterpret_cast<const float4*>(a.norm_w);
    __syncthreads();  // every warp sees the barrier initialised
    pdl_wait();
    if (!a.release_early) pdl_launch_dependents();
    trace_mark(a.trace, 2);
    trace_mark(a.trace, 3);

    // ---- x: straight into registers, or normalised into shared memory ---------
    uint32_t ax[kSteps][4];
    if (kDirect) {
        // lane (g, t): rows g and g + 8, columns 4 t .. 4 t + 3 of each step of 16
        const int g = lane >> 2, t4 = (lane & 3) * 4;
        const bf16* x0 = a.x + (size_t)(row0 + g) * a.ldx + k_begin + t4;
        const bf16* x1 = x0 + (size_t)8 * a.ldx;
        const bool in_a = row0 + g < a.M, in_b = row0 + g + 8 < a.M;
#pragma unroll
        for (int s = 0; s < kSteps; ++s) {
            const bool in_k = k_begin + s * 16 < k_end;
            const uint2 zero = make_uint2(0u, 0u);
            const uint2 va = in_k && in_a ? *reinterpret_cast<const uint2*>(x0 + s * 16) : zero;
            const uint2 vb = in_k && in_b ? *reinterpret_cast<const uint2*>(x1 + s * 16) : zero;
            ax[s][0] = va.x;
            ax[s][1] = vb.x;
            ax[s][2] = va.y;
            ax[s][3] = vb.y;
        }
        if (kScaled) {
            // sixteen threads to a row add up its shares, each in a fixed order
            const int r = threadIdx.x >> 4, part = threadIdx.x & 15;
            const bool live = row0 + r < a.M;
            const float* parts = a.ss_parts + (size_t)(live ? row0 + r : 0) * a.ss_units;
            float ss = 0.f;
            for (int j0 = part; j0 < a.ss_units; j0 += 16 * 8) {
                float sv8[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) sv8[j] = live && j0 + 16 * j < a.ss_units ? parts[j0 + 16 * j] : 0.f;
#pragma unroll
                for (int j = 0; j < 8; ++j) ss += sv8[j];
            }
            ss = half_warp_sum(ss);
            if (part == 0) row_scale[r] = 1.0f / sqrtf(ss * (1.0f / (float)K) + a.eps);
        }
    } else if (few) {
        // a warp to a row (row 8, of zeros, is warp 0's second)
        for (int r = warp; r < xrows; r += WARPS) {
            const int m = row0 + r;
            if (r < 8 && m < a.M) {
                const float4* h4 = reinterpret_cast<const float4*>(a.hidden + (size_t)(a.rows ? a.rows[m] : m) * K);
                if (k4 <= 32 * NWF) {
                    float4 hv[NWF];
                    float ss = 0.f;
#pragma unroll
                    for (int j = 0; j < NWF; ++j) {
                        int c = lane + 32 * j;
                        hv[j] = c < k4 ? h4[c] : make_float4(0.f, 0.f, 0.f, 0.f);
                    }
#pragma unroll
                    for (int j = 0; j < NWF; ++j) {
                        ss = fmaf(hv[j].x, hv[j].x, ss);
                        ss = fmaf(hv[j].y, hv[j].y, ss);
                        ss = fmaf(hv[j].z, hv[j].z, ss);
                        ss = fmaf(hv[j].w, hv[j].w, ss);
                    }
                    ss = warp_sum(ss);
                    const float sc = 1.0f / sqrtf(ss * (1.0f / (float)K) + a.eps);
#pragma unroll
                    for (int j = 0; j < NWF; ++j) {
                        int c = lane + 32 * j;
                        if (c < k4)
                            store4(xs + (size_t)r * KP + c * 4,
                                   make_float4((hv[j].x * sc) * nw[j].x, (hv[j].y * sc) * nw[j].y,
                                               (hv[j].z * sc) * nw[j].z, (hv[j].w * sc) * nw[j].w));
                    }
                } else {
                    const float ss = warp_sum(row_square_sum<32>(h4, k4, lane));
                    const float sc = 1.0f / sqrtf(ss * (1.0f / (float)K) + a.eps);
                    row_scale_store<32>(h4, w4, k4, lane, sc, xs + (size_t)r * KP);
                }
            } else {
                for (int k = lane * 2; k < K; k += 64) *reinterpret_cast<uint32_t*>(xs + (size_t)r * KP + k) = 0u;
            }
        }
        __syncthreads();
    } else {
        // half a warp to a row: the warp's two rows are in flight together
        const int hl = lane & 15;
        const int r = warp * 2 + (lane >> 4);
        const int m = row0 + r;
        const bool in_regs = k4 <= 16 * NW;
        const bool live = m < a.M;  // (the shuffles below name every lane: no lane leaves early)
        const float4* h4 = reinterpret_cast<const float4*>(a.hidden + (live ? (size_t)(a.rows ? a.rows[m] : m) * K : 0));
        float4 hv[NW];
        float ss = 0.f;
        if (in_regs) {
#pragma unroll
            for (int j = 0; j < NW; ++j) {
                int c = hl + 16 * j;
                hv[j] = live && c < k4 ? h4[c] : make_float4(0.f, 0.f, 0.f, 0.f);
            }
#pragma unroll
            for (int j = 0; j < NW; ++j) {
                ss = fmaf(hv[j].x, hv[j].x, ss);
                ss = fmaf(hv[j].y, hv[j].y, ss);
                ss = fmaf(hv[j].z, hv[j].z, ss);
                ss = fmaf(hv[j].w, hv[j].w, ss);
            }
        } else if (live) {
            ss = row_square_sum<16>(h4, k4, hl);
        }
        ss = half_warp_sum(ss);
        const float sc = 1.0f / sqrtf(ss * (1.0f / (float)K) + a.eps);
        if (!live) {
            for (int k = hl * 2; k < K; k += 32) *reinterpret_cast<uint32_t*>(xs + (size_t)r * KP + k) = 0u;
        } else if (in_regs) {
#pragma unroll
            for (int j = 0; j < NW; ++j) {
                int c = hl + 16 * j;
                if (c < k4) {
                    const float4 g = w4[c];
                    store4(xs + (size_t)r * KP + c * 4,
                           make_float4((hv[j].x * sc) * g.x, (hv[j].y * sc) * g.y,
                                       (hv[j].z * sc) * g.z, (hv[j].w * sc) * g.w));
                }
            }
        } else {
            row_scale_store<16>(h4, w4, k4, hl, sc, xs + (size_t)r * KP);
        }
        __syncthreads();
    }
    trace_mark(a.trace, 4);
    trace_mark(a.trace, 5);

    // ---- products: this warp's columns, all units ----------------------------------
    // (a wait that runs out is flagged; the CTA goes on through its barriers)
    const bool arrived = mbar_wait(&wbar, 0);
    float acc[NU][4];
#pragma unroll
    for (int u = 0; u < NU; ++u)
#pragma unroll
        for (int e = 0; e < 4; ++e) acc[u][e] = 0.f;
    if (kDirect) {
        // the weights in the order of x: lane (g, t) takes columns 4 t .. 4 t + 3 of row g
        const bf16* b_ptr = ws + (size_t)(lane >> 2) * KPW + (lane & 3) * 4;
#pragma unroll
        for (int s = 0; s < kSteps; ++s) {
            const int k0 = k_begin + s * 16;
            if (k0 < k_end) {
                uint2 bw[NU];
#pragma unroll
                for (int u = 0; u < NU; ++u)
                    bw[u] = *reinterpret_cast<const uint2*>(b_ptr + (size_t)u * 8 * KPW + k0);
#pragma unroll
                for (int u = 0; u < NU; ++u) mma_bf16(acc[u], ax[s], bw[u].x, bw[u].y);
            }
        }
    } else {
        // lanes 0-7: weight rows at columns k0..k0+7, lanes 8-15: k0+8..k0+15
        const bf16* b_ptr = ws + (size_t)(lane & 7) * KPW + ((lane >> 3) & 1) * 8;
        // (with the row of zeros, the lanes of rows 8-15 all read it)
        const bf16* a_ptr = xs + (size_t)min(lane & 15, xrows - 1) * KP + (lane >> 4) * 8;
#pragma unroll 2
        for (int k0 = k_begin; k0 < k_end; k0 += 16) {
            uint32_t af[4], bw[NU][2];
            ldmatrix_x4(af, a_ptr + k0);
#pragma unroll
            for (int u = 0; u < NU; ++u) ldmatrix_x2(bw[u][0], bw[u][1], b_ptr + (size_t)u * 8 * KPW + k0);
#pragma unroll
            for (int u = 0; u < NU; ++u) mma_bf16(acc[u], af, bw[u][0], bw[u][1]);
        }
    }
    trace_mark(a.trace, 6);
    trace_mark(a.trace, 7);

    // ---- the warps' partial sums, added in warp order by the unit's warp ----------
    __syncthreads();  // every warp has read its weights: their place is free
#pragma unroll
    for (int u = 0; u < NU; ++u)
#pragma unroll
        for (int e = 0; e < 4; ++e) red[((size_t)(warp * NU + u) * 4 + e) * 32 + lane] = acc[u][e];
    __syncthreads();
    if (epi_warp) {
        float sum[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            float v = red[((size_t)warp * 4 + e) * 32 + lane];
            for (int w = 1; w < WARPS; ++w) v += red[((size_t)(w * NU + warp) * 4 + e) * 32 + lane];
            sum[e] = v;
        }
        if (kScaled) {  // (written before the two barriers above)
            const float s_lo = row_scale[lane >> 2], s_hi = row_scale[(lane >> 2) + 8];
            sum[0] *= s_lo;
            sum[1] *= s_lo;
            sum[2] *= s_hi;
            sum[3] *= s_hi;
        }
        float best_v[2] = {0.f, 0.f};
        int best_i[2] = {-1, -1};
        epi_finish<EPI>(a, unit0 + warp, row0, lane, sum, pre, true, best_v, best_i);
    }
    if (!arrived && lane == 0 && a.status) atomicExch(a.status, 2);
    trace_mark(a.trace, 1);
}

static size_t rowtile_smem(int M, int nu, int K, int pro) {
    size_t operands = (size_t)nu * 8 * rowtile_w_stride(K, pro) * sizeof(bf16);
    if (pro == PRO_NORM)
        operands += (size_t)rowtile_x_rows(M) * (K + 8) * sizeof(bf16) + (M > 8 ? (size_t)K * sizeof(float) : 0);
    size_t sums = (size_t)kRowtileWarps * nu * 4 * 32 * sizeof(float);
    return operands > sums ? operands : sums;
}

// Units per CTA for a product of these sizes, or 0 when this kernel does not take it:
// at most eight tiles of rows, K in steps of 16 (at most 1,536 without the norm: a
// warp's share of x lives in registers), no ARGMAX epilogue, and every CTA resident at
// once, so that all of W is asked for before the wait.
int gemv_rowtile_units(int M, int N, int K, int epilogue, int pro, int sm_count) {
    if (M <= 0 || M > 128 || K <= 0 || K % 16 || N <= 0 || N % 8) return 0;
    if (epilogue == EPI_ARGMAX) return 0;
    if (pro != PRO_NORM && K > rowtile_direct_steps(true) * 16 * kRowtileWarps) return 0;
    if (pro == PRO_SCALED && epilogue != EPI_QKV && epilogue != EPI_GATED) return 0;
    const bool longk = pro != PRO_NORM && K > rowtile_direct_steps(false) * 16 * kRowtileWarps;
    const int sms = sm_count > 0 ? sm_count : 148;
    const int mtiles = (M + 15) / 16, units = N / 8;
    // With one tile of rows: few units per CTA, and CTAs for at most one and a half SMs'
    // worth, which leaves room on the SMs for the kernels before and after.  With more:
    // as many units as tiles of rows keeps the number of CTAs near the number of units, and
    // the bytes of x that a CTA fetches after the wait below those of W.
    // (one tile of rows: two units a CTA from 64 units on measured as one unit at batch 8 of
    // the 135M shape and 3 % better at batch 1: fewer CTAs in the way of the attention kernel's)
    static const int min_units = getenv("NNIS_ROWTILE_MIN_UNITS") ? atoi(getenv("NNIS_ROWTILE_MIN_UNITS")) : 0;
    const int first = mtiles >= 3 ? 4 : mtiles == 2 ? 2 : min_units > 0 ? min_units : units >= 64 ? 2 : 1;
    for (int nu = first; nu <= 4; nu *= 2) {
        size_t smem = rowtile_smem(M, nu, K, pro);
        if (smem > 200 * 1024) continue;
        int fit = (int)((220 * 1024) / (smem + 1024));
        if (fit > rowtile_ctas_per_sm(epilogue, pro, longk)) fit = rowtile_ctas_per_sm(epilogue, pro, longk);
        long ctas = (long)mtiles * ((units + nu - 1) / nu);
        long room = mtiles == 1 ? (long)sms * 3 / 2 : (long)sms * fit;
        if (fit >= 1 && ctas <= room && ctas <= (long)sms * fit) return nu;
    }
    return 0;
}

template <int EPI, int PRO, int NU, bool LONGK>
static int launch_rowtile_final(const GemvArgs& a, bool pdl, cudaStream_t stream) {
    auto kernel = gemv_rowtile_kernel<EPI, PRO, NU, LONGK>;
    const size_t smem = rowtile_smem(a.M, NU, a.K, PRO);
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(((a.N >> 3) + NU - 1) / NU, (a.M + 15) / 16);
    cfg.blockDim = dim3(kRowtileWarps * 32);
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

template <int EPI, int PRO>
static int launch_rowtile_units(const GemvArgs& a, int nu, bool pdl, cudaStream_t stream) {
    // (with the norm in front x is in shared memory: one variant for every K)
    const bool longk = PRO != PRO_NORM && a.K > rowtile_direct_steps(false) * 16 * kRowtileWarps;
    if (longk) {
        if (nu == 1) return launch_rowtile_final<EPI, PRO, 1, PRO != PRO_NORM>(a, pdl, stream);
        if (nu == 2) return launch_rowtile_final<EPI, PRO, 2, PRO != PRO_NORM>(a, pdl, stream);
        if (nu == 4) return launch_rowtile_final<EPI, PRO, 4, PRO != PRO_NORM>(a, pdl, stream);
    } else {
        if (nu == 1) return launch_rowtile_final<EPI, PRO, 1, false>(a, pdl, stream);
        if (nu == 2) return launch_rowtile_final<EPI, PRO, 2, false>(a, pdl, stream);
        if (nu == 4) return launch_rowtile_final<EPI, PRO, 4, false>(a, pdl, stream);
    }
    return NNIS_ERR_UNSUPPORTED;
}

// `nu` from gemv_rowtile_units for the same sizes.
int gemv_launch_rowtile(const GemvArgs& a, int epi, int pro, int nu, bool pdl, cudaStream_t stream) {
#define NNIS_ROWTILE(EPI, PRO) return launch_rowtile_units<EPI, PRO>(a, nu, pdl, stream)
    if (epi == EPI_QKV && pro == PRO_NORM) NNIS_ROWTILE(EPI_QKV, PRO_NORM);
    if (epi == EPI_QKV && pro == PRO_PLAIN) NNIS_ROWTILE(EPI_QKV, PRO_PLAIN);
    if (epi == EPI_GATED && pro == PRO_NORM) NNIS_ROWTILE(EPI_GATED, PRO_NORM);
    if (epi == EPI_GATED && pro == PRO_PLAIN) NNIS_ROWTILE(EPI_GATED, PRO_PLAIN);
    if (epi == EPI_QKV && pro == PRO_SCALED) NNIS_ROWTILE(EPI_QKV, PRO_SCALED);
    if (epi == EPI_GATED && pro == PRO_SCALED) NNIS_ROWTILE(EPI_GATED, PRO_SCALED);
    if (epi == EPI_ADD_F32 && pro == PRO_PLAIN) NNIS_ROWTILE(EPI_ADD_F32, PRO_PLAIN);
    if (epi == EPI_STORE && pro == PRO_PLAIN) NNIS_ROWTILE(EPI_STORE, PRO_PLAIN);
    if (epi == EPI_STORE_F32 && pro == PRO_PLAIN) NNIS_ROWTILE(EPI_STORE_F32, PRO_PLAIN);
    if (epi == EPI_STORE_F32 && pro == PRO_NORM) NNIS_ROWTILE(EPI_STORE_F32, PRO_NORM);
#undef NNIS_ROWTILE
    return NNIS_ERR_UNSUPPORTED;
}

}  // namespace nnis
