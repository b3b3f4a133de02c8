// bfloat16 matrix product on the fifth-generation tensor cores of sm_100a:
// C[M, N] (op)= A[M, K] . W[N, K]^T + bias, float32 accumulation in tensor memory.
//
// One CTA computes a 128 x BN tile (BN = 64 or 128).  Its six warps have fixed
// roles:
//   warp 0  one lane issues TMA tile loads (cp.async.bulk.tensor, 128-byte
//           swizzle) of A, one, two or four slices of 64 columns of K per stage, into a
//           ring of shared memory stages, each guarded by a "full" and an "empty"
//           mbarrier; lane 0 of warp 2 does the same for W;
//   warp 1  allocates tensor memory, and one lane issues tcgen05.mma
//           (kind::f16, M = 128, N = BN, K = 16) four times per slice from shared
//           memory descriptors, then tcgen05.commit to hand the stage back and,
//           after the last one, to tell the epilogue that the accumulator is done;
//   warps 2-5  read the accumulator with tcgen05.ld (each warp its own 32 lanes
//           of tensor memory = 32 rows of the tile), add the bias, and hand the
//           tile through shared memory to a TMA store (bfloat16 or float32) or a
//           TMA addition into a float32 destination.
// Rows and columns beyond M, N and K are zero-filled by TMA on the way in and
// clipped on the way out, so any M and N and any K that is a multiple of 8 work.
//
// Every wait is bounded: a wait that runs out sets a status word and an abort
// flag that the other roles see; all warps still meet at the end, and tensor
// memory is always freed.
// NNIS computes the same product on CUDA cores: crates/nnis-kernels/src/gemm.rs:16-64.
#include "tcgen05_helpers.cuh"

namespace nnis {

constexpr int kBM = 128;
constexpr int kBK = 64;          // 64 bfloat16 = one 128-byte swizzle row
constexpr int kUmmaK = 16;
constexpr int kMaxKSplits = 4;   // CTAs that may share a tile of the adding product

enum { GEMM_STORE = 0, GEMM_STORE_F32 = 1, GEMM_ADD_F32 = 2, GEMM_GATED = 3, GEMM_QKV = 4 };

struct GemmArgs {
    const float* bias;
    void* out;
    int M, N, K;
    int* status;
    int out_by_tma;  // the output's rows start on 16-byte boundaries: tiles leave through shared memory
    // GEMM_ADD_F32 with few tiles and a long K: CTA (x, y, z) takes the z-th run of k-blocks,
    // leaves its sums in `split_scratch` ([tile, split, 128 rows, BN] float32) and takes a
    // ticket; the CTA of a tile that arrives last adds the splits' sums in the order of
    // the splits (deterministic) and adds the result into the output
    int k_splits;
    float* split_scratch;
    unsigned* split_tickets;  // one per tile, zero between launches
    // GEMM_QKV: rotate-half RoPE of q and k heads at each row's position, q to
    // `out` [M, nq * d], k and v into the paged cache (one head per column tile)
    const int* token_pos;
    const int* token_seq;
    const int* page_table;
    int table_cols;
    const float* cos_t;
    const float* sin_t;
    bf16* k_cache;
    bf16* v_cache;
    int nq, nkv, d, page_size;
    unsigned long long* trace;  // this launch's slot of the step's timeline, or null
};

// Two CTAs share an SM when their stages leave room for it.
__host__ __device__ constexpr int gemm_ctas_per_sm(int bn, int stages, int mode, int ksub) {
    return stages * ksub * (kBM + (mode == GEMM_GATED ? 2 : 1) * bn) * kBK * 2 <= 110 * 1024 ? 2 : 1;
}
// A warp that is alone on its scheduler runs every instruction at full latency, so
// a CTA that has its SM alone brings eight epilogue warps, two per quarter of the
// rows, each taking every other chunk of 32 columns; with two CTAs per SM the four
// epilogue warps of each leave the registers for both.  The wide gate/up tile (192 + 192
// columns, two special-function instructions a value) brings sixteen: its epilogue went
// from 4.0 to 2.4 us of arithmetic at 2,048 rows.
__host__ __device__ constexpr int gemm_threads(int bn, int stages, int mode, int ksub) {
    return gemm_ctas_per_sm(bn, stages, mode, ksub) == 1 ? (bn == 192 ? 576 : 320) : 192;
}

// MODE GEMM_GATED: W holds gate rows then up rows ([2 I, K]); the CTA multiplies
// A by a gate tile and by the matching up tile into two accumulators and writes
// bf16(silu(gate) * up) to out [M, I].  MODE GEMM_QKV: a tile holds whole heads
// (BN = 128: two heads of 64 or one of 128).
// SPLIT: K cut among the CTAs of a tile (GemmArgs::k_splits), a build of its own so that
// the others carry none of it.
template <int BN, int STAGES, int MODE, int KSUB, bool SPLIT = false>
__global__ void __launch_bounds__(gemm_threads(BN, STAGES, MODE, KSUB), gemm_ctas_per_sm(BN, STAGES, MODE, KSUB))
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w,
               const __grid_constant__ CUtensorMap map_out, GemmArgs g) {
    trace_mark(g.trace, 0);
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    // the swizzle pattern follows address bits: tiles start on 1024-byte boundaries
    unsigned char* base = reinterpret_cast<unsigned char*>(
        (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    constexpr int NB = MODE == GEMM_GATED ? 2 : 1;  // B tiles (and accumulators) per stage
    constexpr int kEpiWarps = gemm_threads(BN, STAGES, MODE, KSUB) / 32 - 2;
    constexpr int kColStep = 32 * (kEpiWarps / 4);  // columns between two chunks of one warp
    constexpr uint32_t kBytesA = kBM * kBK * 2, kBytesB = BN * kBK * 2;
    // tensor memory comes in powers of two of columns
    constexpr uint32_t kTmemCols = NB * BN <= 64 ? 64 : NB * BN <= 128 ? 128 : NB * BN <= 256 ? 256 : 512;
    // a stage holds KSUB slices of 64 columns of K: [KSUB] A tiles, then [KSUB][NB] W tiles
    constexpr uint32_t kStageA = KSUB * kBytesA, kStageB = KSUB * NB * kBytesB;
    unsigned char* tile_a = base;
    unsigned char* tile_b = base + (size_t)STAGES * kStageA;
    __shared__ __align__(8) uint64_t full_bar[STAGES], empty_bar[STAGES], acc_bar, staged_bar, split_bar, split_done;
    __shared__ uint32_t tmem_base_s;
    __shared__ int split_last;
    __shared__ volatile int abort_flag;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int m0 = blockIdx.y * kBM, n0 = blockIdx.x * BN;
    const int k_slices = (g.K + kBK - 1) / kBK;
    const int k_blocks_all = (k_slices + KSUB - 1) / KSUB;
    // this CTA's run of k-blocks (all of them without a split of K)
    const int kb_per = SPLIT ? (k_blocks_all + g.k_splits - 1) / g.k_splits : k_blocks_all;
    const int kb_first = SPLIT ? (int)blockIdx.z * kb_per : 0;
    const int k_blocks = SPLIT ? max(0, min(kb_per, k_blocks_all - kb_first)) : k_blocks_all;
    const int inter = g.N >> 1;  // GEMM_GATED: columns of the output

    if (threadIdx.x == 32) {
        prefetch_tensormap(&map_a);
        prefetch_tensormap(&map_w);
        if (g.out_by_tma) prefetch_tensormap(&map_out);
    }
    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(&full_bar[s], 2);   // the two loaders
            mbar_init(&empty_bar[s], 1);
        }
        mbar_init(&acc_bar, 1);
        mbar_init(&staged_bar, kEpiWarps);
        mbar_init(&split_bar, kEpiWarps);
        mbar_init(&split_done, 1);
        abort_flag = 0;
        mbar_fence_init();
    }
    if (warp == 1) tmem_alloc(&tmem_base_s, kTmemCols);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_acc = tmem_base_s;

    // Issuing a TMA load costs its thread about 130 cycles, so A and W each have a
    // loader of their own: lane 0 of warp 0 and lane 0 of warp 2 (which joins the
    // epilogue afterwards).  Each announces its own bytes; a stage is full when both
    // have arrived and all bytes are there.
    auto load_stage = [&](bool loads_a, int kb) {
        const int s = kb % STAGES;
        // (slices beyond K arrive as zeros and are not multiplied)
        mbar_expect_tx(&full_bar[s], loads_a ? kStageA : kStageB);
#pragma unroll
        for (int h = 0; h < KSUB; ++h) {
            const int k0 = ((kb_first + kb) * KSUB + h) * kBK;
            if (loads_a) {
                tma_load_2d(tile_a + (size_t)s * kStageA + (size_t)h * kBytesA, &map_a, k0, m0,
                            &full_bar[s]);
            } else {
                unsigned char* b_dst = tile_b + (size_t)s * kStageB + (size_t)h * NB * kBytesB;
                tma_load_2d(b_dst, &map_w, k0, n0, &full_bar[s]);
                if (NB == 2) tma_load_2d(b_dst + kBytesB, &map_w, k0, inter + n0, &full_bar[s]);
            }
        }
    };
    // A depends on the kernel before this one; W does not: the first stages of W are
    // asked for before the wait, under that kernel's tail
    int w_ahead = 0;
    if (warp == 2 && lane == 0)
        for (; w_ahead < k_blocks && w_ahead < STAGES; ++w_ahead) load_stage(false, w_ahead);
    pdl_wait();
    pdl_launch_dependents();
    trace_mark(g.trace, 2);
    trace_mark(g.trace, 3);

    if (lane == 0 && (warp == 0 || warp == 2)) {
        const bool loads_a = warp == 0;
        for (int kb = loads_a ? 0 : w_ahead; kb < k_blocks; ++kb) {
            int s = kb % STAGES;
            if (kb >= STAGES && !mbar_wait(&empty_bar[s], (uint32_t)(kb / STAGES - 1) & 1u)) {
                abort_flag = 1;
                break;
            }
            if (abort_flag) break;
            load_stage(loads_a, kb);
        }
    }
    __syncwarp();
    if (warp == 0) {
        // nothing more: the loader of A waits for the end with its warp
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr uint32_t idesc = instr_desc(kBM, BN);
            const uint64_t desc_a0 = smem_desc_k128(smem_addr(tile_a));
            const uint64_t desc_b0 = smem_desc_k128(smem_addr(tile_b));
            bool ok = true;
            for (int kb = 0; kb < k_blocks; ++kb) {
                int s = kb % STAGES;
                if (!mbar_wait(&full_bar[s], (uint32_t)(kb / STAGES) & 1u) || abort_flag) {
                    ok = false;
                    break;
                }
                tc_fence_after();
                if (kb == 0) {  // the first operands have arrived
                    trace_mark_here(g.trace, 4);
                    trace_mark_here(g.trace, 5);
                }
#pragma unroll
                for (int h = 0; h < KSUB; ++h) {
                    if ((kb_first + kb) * KSUB + h >= k_slices) break;
                    const uint64_t da = desc_advance(desc_a0, (uint32_t)s * kStageA + h * kBytesA);
                    const uint64_t db = desc_advance(desc_b0, (uint32_t)s * kStageB + h * NB * kBytesB);
#pragma unroll
                    for (int k = 0; k < kBK / kUmmaK; ++k) {
                        // 16 columns of K further along the swizzled row: 32 bytes
                        tc_mma(tmem_acc, desc_advance(da, k * kUmmaK * 2), desc_advance(db, k * kUmmaK * 2),
                               idesc, (kb | h | k) != 0);
                        if (NB == 2)
                            tc_mma(tmem_acc + BN, desc_advance(da, k * kUmmaK * 2),
                                   desc_advance(db, kBytesB + k * kUmmaK * 2), idesc, (kb | h | k) != 0);
                    }
                }
                tc_commit(&empty_bar[s]);  // the stage is free once these MMAs have read it
            }
            if (!ok) abort_flag = 1;
            tc_commit(&acc_bar);  // arrives when all MMAs above are complete (also after an abort)
        }
    } else {
        // epilogue: warp w reads tensor-memory lanes 32 (w % 4) .. + 31 = tile rows
        const int quarter = warp & 3;
        const int c_first = 32 * ((warp - 2) >> 2);  // this warp's first chunk of columns
        const int row = quarter * 32 + lane;
        const int m = m0 + row;
        const uint32_t lane_base = tmem_acc + ((uint32_t)(quarter * 32) << 16);
        // GEMM_QKV: what the epilogue needs from global memory (the row's position,
        // its cache page, the angles of this warp's first unit) is fetched while the
        // products run
        int pos = -1, page = 0;
        float cs[32], sn[32];
        if (MODE == GEMM_QKV) {
            pos = m < g.M ? g.token_pos[m] : -1;
            if (pos >= 0 && g.nkv > 0)
                page = g.page_table[(size_t)g.token_seq[m] * g.table_cols + pos / g.page_size];
            const int half = g.d / 2, c0 = (((warp - 2) >> 2) % (half / 32)) * 32;
            if (pos >= 0 && g.sin_t) {
                const float4* c4 = reinterpret_cast<const float4*>(g.cos_t + (size_t)pos * half + c0);
                const float4* s4 = reinterpret_cast<const float4*>(g.sin_t + (size_t)pos * half + c0);
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    float4 cv = c4[i], sv = s4[i];
                    cs[i * 4] = cv.x; cs[i * 4 + 1] = cv.y; cs[i * 4 + 2] = cv.z; cs[i * 4 + 3] = cv.w;
                    sn[i * 4] = sv.x; sn[i * 4 + 1] = sv.y; sn[i * 4 + 2] = sv.z; sn[i * 4 + 3] = sv.w;
                }
            }
        }
        bool ok = mbar_wait(&acc_bar, 0);
        if (warp == 2 && lane == 0) {  // the products are complete
            trace_mark_here(g.trace, 6);
            trace_mark_here(g.trace, 7);
        }
        ok = __all_sync(0xffffffffu, ok) && !abort_flag;
        if (!ok) {
            abort_flag = 1;
        } else if (MODE == GEMM_QKV) {
            tc_fence_after();
            // The tile holds BN / d whole heads; this thread holds one row of each.
            // Columns j and j + d/2 of a head are a rotation pair, in chunks c0 and
            // c0 + d/2.  The units of work (head of the tile, chunk) are dealt to the
            // warps that share this quarter of the rows.
            const int d = g.d, half = d / 2, chunks = half / 32;
            const int first_unit = (warp - 2) >> 2;
            int angles_of = first_unit % chunks;  // the chunk whose cos and sin are in registers
#pragma unroll 1
            for (int unit = first_unit; unit < (BN / d) * chunks; unit += kEpiWarps / 4) {
                const int hh = unit / chunks, c0 = (unit % chunks) * 32;
                const int head = n0 / d + hh;
                if (head >= g.nq + 2 * g.nkv) break;
                const bool is_q = head < g.nq, is_v = head >= g.nq + g.nkv;
                const uint32_t cols = (uint32_t)(hh * d + c0);
                uint32_t va[32], vb[32];
                tmem_load32_issue(lane_base + cols, va);
                tmem_load32_issue(lane_base + cols + (uint32_t)half, vb);
                tmem_load_wait();
                if (pos < 0) continue;
                bf16* dst;
                if (is_q) {
                    dst = reinterpret_cast<bf16*>(g.out) + ((size_t)m * g.nq + head) * d;
                } else {
                    int hk = is_v ? head - g.nq - g.nkv : head - g.nq;
                    dst = (is_v ? g.v_cache : g.k_cache) +
                          ((size_t)(page * g.nkv + hk) * g.page_size + (pos % g.page_size)) * d;
                }
                const int nb = head * d + c0;  // column of W's rows, for the bias
                uint32_t oa[16], ob[16];
                if (g.sin_t && !is_v && (unit % chunks) != angles_of) {
                    angles_of = unit % chunks;
                    const float4* c4 = reinterpret_cast<const float4*>(g.cos_t + (size_t)pos * half + c0);
                    const float4* s4 = reinterpret_cast<const float4*>(g.sin_t + (size_t)pos * half + c0);
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        float4 cv = c4[i], sv = s4[i];
                        cs[i * 4] = cv.x; cs[i * 4 + 1] = cv.y; cs[i * 4 + 2] = cv.z; cs[i * 4 + 3] = cv.w;
                        sn[i * 4] = sv.x; sn[i * 4 + 1] = sv.y; sn[i * 4 + 2] = sv.z; sn[i * 4 + 3] = sv.w;
                    }
                }
#pragma unroll
                for (int i = 0; i < 32; i += 2) {
                    float a0 = __uint_as_float(va[i]), a1 = __uint_as_float(va[i + 1]);
                    float b0 = __uint_as_float(vb[i]), b1 = __uint_as_float(vb[i + 1]);
                    if (g.bias) {
                        a0 += g.bias[nb + i];
                        a1 += g.bias[nb + i + 1];
                        b0 += g.bias[nb + half + i];
                        b1 += g.bias[nb + half + i + 1];
                    }
                    // q, k and v are bfloat16 before the rotation, as in the unfused path
                    a0 = __bfloat162float(__float2bfloat16_rn(a0));
                    a1 = __bfloat162float(__float2bfloat16_rn(a1));
                    b0 = __bfloat162float(__float2bfloat16_rn(b0));
                    b1 = __bfloat162float(__float2bfloat16_rn(b1));
                    if (g.sin_t && !is_v) {
                        float c_0 = cs[i], c_1 = cs[i + 1], s_0 = sn[i], s_1 = sn[i + 1];
                        float r0 = a0 * c_0 - b0 * s_0, r1 = a1 * c_1 - b1 * s_1;
                        b0 = b0 * c_0 + a0 * s_0;
                        b1 = b1 * c_1 + a1 * s_1;
                        a0 = r0;
                        a1 = r1;
                    }
                    __nv_bfloat162 pa = __floats2bfloat162_rn(a0, a1), pb = __floats2bfloat162_rn(b0, b1);
                    oa[i >> 1] = *reinterpret_cast<uint32_t*>(&pa);
                    ob[i >> 1] = *reinterpret_cast<uint32_t*>(&pb);
                }
#pragma unroll
                for (int i = 0; i < 16; i += 4) {
                    *reinterpret_cast<uint4*>(dst + c0 + i * 2) = make_uint4(oa[i], oa[i + 1], oa[i + 2], oa[i + 3]);
                    *reinterpret_cast<uint4*>(dst + c0 + half + i * 2) =
                        make_uint4(ob[i], ob[i + 1], ob[i + 2], ob[i + 3]);
                }
            }
        } else {
            tc_fence_after();
            // Each thread owns one row.  The tile leaves through shared memory (the
            // ring is idle by now): rows of 128 bytes, 16-byte units swizzled as the
            // output's tensor map says, then one TMA store per 128-byte-wide box, or
            // a TMA addition into the float32 destination, which spares reading it.
            // TMA clips rows and columns beyond M and N.  An output whose rows do not
            // start on 16-byte boundaries is written element by element.
            const int out_cols = MODE == GEMM_GATED ? inter : g.N;
            constexpr bool kOut16 = MODE == GEMM_STORE || MODE == GEMM_GATED;
            constexpr int kBoxCols = kOut16 ? 64 : 32;
            unsigned char* stage_row = base + (size_t)row * 128;
            // With K split among CTAs: this CTA's sums to scratch, a ticket, and only the CTA
            // of the tile that arrives last goes on, with the sums of all splits.
            constexpr bool split = SPLIT && MODE == GEMM_ADD_F32;
            const size_t tile_id = (size_t)blockIdx.y * gridDim.x + blockIdx.x;
            float* tile_sums = g.split_scratch + (tile_id * (size_t)g.k_splits * kBM + row) * BN;
            bool finishes = true;
            if constexpr (split) {
                float* mine = tile_sums + (size_t)blockIdx.z * kBM * BN;
#pragma unroll 1
                for (int c0 = c_first; c0 < BN; c0 += kColStep) {
                    uint32_t v[32];
                    tmem_load32_issue(lane_base + (uint32_t)c0, v);
                    tmem_load_wait();
                    if (m < g.M) {  // (rows beyond M are never read)
#pragma unroll
                        for (int j = 0; j < 8; ++j)
                            __stcg(reinterpret_cast<float4*>(mine + c0) + j,
                                   make_float4(__uint_as_float(v[j * 4]), __uint_as_float(v[j * 4 + 1]),
                                               __uint_as_float(v[j * 4 + 2]), __uint_as_float(v[j * 4 + 3])));
                    }
                }
                // every epilogue warp has written (bounded waits, as everywhere: a warp that
                // gave up earlier must not leave the others waiting for ever)
                __threadfence();
                __syncwarp();
                if (lane == 0) mbar_arrive(&split_bar);
                if (threadIdx.x == 64) {
                    split_last = 0;
                    if (mbar_wait(&split_bar, 0)) {
                        unsigned old;
                        asm volatile("atom.add.acq_rel.gpu.global.u32 %0, [%1], 1;"
                                     : "=r"(old) : "l"(g.split_tickets + tile_id) : "memory");
                        split_last = old == (unsigned)g.k_splits - 1u;
                        if (split_last) g.split_tickets[tile_id] = 0u;  // (every split has arrived)
                    } else {
                        abort_flag = 1;
                    }
                    mbar_arrive(&split_done);
                }
                if (!mbar_wait(&split_done, 0)) abort_flag = 1;
                finishes = split_last != 0 && !abort_flag;
            }
#pragma unroll 1
            for (int c0 = c_first; c0 < BN && finishes; c0 += kColStep) {
                uint32_t v[32], u[32];
                if constexpr (split) {
                    // the splits' sums of this row: all asked for at once (one trip to L2),
                    // added in the order of the splits
                    float4 part[kMaxKSplits][8];
#pragma unroll
                    for (int z = 0; z < kMaxKSplits; ++z) {
                        const float4* src = reinterpret_cast<const float4*>(tile_sums + (size_t)z * kBM * BN + c0);
#pragma unroll
                        for (int j = 0; j < 8; ++j)
                            part[z][j] = z < g.k_splits && m < g.M ? __ldcg(src + j) : make_float4(0.f, 0.f, 0.f, 0.f);
                    }
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        float4 sum = part[0][j];
#pragma unroll
                        for (int z = 1; z < kMaxKSplits; ++z) {
                            sum.x += part[z][j].x;
                            sum.y += part[z][j].y;
                            sum.z += part[z][j].z;
                            sum.w += part[z][j].w;
                        }
                        v[j * 4] = __float_as_uint(sum.x);
                        v[j * 4 + 1] = __float_as_uint(sum.y);
                        v[j * 4 + 2] = __float_as_uint(sum.z);
                        v[j * 4 + 3] = __float_as_uint(sum.w);
                    }
                } else {
                    tmem_load32_issue(lane_base + (uint32_t)c0, v);
                    if constexpr (MODE == GEMM_GATED) tmem_load32_issue(lane_base + (uint32_t)(BN + c0), u);
                    tmem_load_wait();
                }
                const int nb = n0 + c0;
                float f[32];
                if constexpr (MODE == GEMM_GATED) {
#pragma unroll
                    for (int i = 0; i < 32; ++i) {
                        float gv = __uint_as_float(v[i]), uv = __uint_as_float(u[i]);
                        if (g.bias && nb + i < inter) {
                            gv += g.bias[nb + i];
                            uv += g.bias[inter + nb + i];
                        }
                        // silu(g) * u with the two approximate instructions (2^x and 1/x,
                        // relative error about 1e-7 each): the exact forms cost the
                        // epilogue twice the time of the products
                        float e, r;
                        asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(gv * -1.4426950408889634f));
                        asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(1.0f + e));
                        f[i] = gv * r * uv;
                    }
                } else {
#pragma unroll
                    for (int i = 0; i < 32; ++i)
                        f[i] = __uint_as_float(v[i]) + ((g.bias && nb + i < g.N) ? g.bias[nb + i] : 0.f);
                }
                if (g.out_by_tma) {
                    unsigned char* box = stage_row + (size_t)(c0 / kBoxCols) * (kBM * 128);
                    if (kOut16) {
                        const int u0 = (c0 % 64) / 8;
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            uint32_t w[4];
#pragma unroll
                            for (int e = 0; e < 4; ++e) {
                                __nv_bfloat162 pk = __floats2bfloat162_rn(f[j * 8 + 2 * e], f[j * 8 + 2 * e + 1]);
                                w[e] = *reinterpret_cast<uint32_t*>(&pk);
                            }
                            *reinterpret_cast<uint4*>(box + (((u0 + j) ^ (row & 7)) << 4)) =
                                make_uint4(w[0], w[1], w[2], w[3]);
                        }
                    } else {
#pragma unroll
                        for (int j = 0; j < 8; ++j)
                            *reinterpret_cast<float4*>(box + ((j ^ (row & 7)) << 4)) =
                                make_float4(f[j * 4], f[j * 4 + 1], f[j * 4 + 2], f[j * 4 + 3]);
                    }
                } else if (m < g.M) {
                    const size_t off = (size_t)m * out_cols + nb;
#pragma unroll
                    for (int i = 0; i < 32; ++i) {
                        if (nb + i < out_cols) {
                            if (kOut16)
                                reinterpret_cast<bf16*>(g.out)[off + i] = __float2bfloat16_rn(f[i]);
                            else if (MODE == GEMM_STORE_F32)
                                reinterpret_cast<float*>(g.out)[off + i] = f[i];
                            else
                                reinterpret_cast<float*>(g.out)[off + i] += f[i];
                        }
                    }
                }
            }
            if (g.out_by_tma && finishes) {
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                __syncwarp();
                if (lane == 0) mbar_arrive(&staged_bar);  // every epilogue warp
                if (threadIdx.x == 64 && !mbar_wait(&staged_bar, 0)) {
                    abort_flag = 1;
                } else if (threadIdx.x == 64) {
#pragma unroll 1
                    for (int c0 = 0; c0 < BN && n0 + c0 < out_cols; c0 += kBoxCols) {
                        const unsigned char* src = base + (size_t)(c0 / kBoxCols) * (kBM * 128);
                        if (MODE == GEMM_ADD_F32) tma_add_2d(&map_out, n0 + c0, m0, src);
                        else tma_store_2d(&map_out, n0 + c0, m0, src);
                    }
                    tma_store_commit_wait();
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_acc, kTmemCols);
    }
    if (threadIdx.x == 0 && abort_flag && g.status) atomicExch(g.status, 3);
    trace_mark(g.trace, 1);
}

template <int BN, int STAGES, int MODE, int KSUB, bool SPLIT = false>
static int launch_gemm_tc(const CUtensorMap& ma, const CUtensorMap& mw, const CUtensorMap& mo,
                          const GemmArgs& g, bool pdl,
                          cudaStream_t stream) {
    constexpr int NB = MODE == GEMM_GATED ? 2 : 1;
    size_t smem = (size_t)STAGES * KSUB * (kBM + NB * BN) * kBK * 2 + 1024;
    auto kernel = gemm_tc_kernel<BN, STAGES, MODE, KSUB, SPLIT>;
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    int n_cols = MODE == GEMM_GATED ? g.N / 2 : g.N;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((n_cols + BN - 1) / BN, (g.M + kBM - 1) / kBM, g.k_splits);
    cfg.blockDim = dim3(gemm_threads(BN, STAGES, MODE, KSUB));
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 1 : 0;
    e = cudaLaunchKernelEx(&cfg, kernel, ma, mw, mo, g);
    return e == cudaSuccess ? NNIS_OK : (int)e;
}

// Into how many runs of k-blocks the adding product cuts K: more than one where 64-column
// tiles are fewer than half the SMs and K is long (a decode step of many rows through a
// projection with a long K: the 1.7B shape's down projection at 64 rows has 32 tiles, each
// streaming a megabyte of weights).  Stages hold 256 columns of K here; every run gets at
// least four of them, no run is empty.
static int gemm_k_splits(long tiles64, int K, int sms) {
    const int k_blocks = (K + 4 * kBK - 1) / (4 * kBK);
    if (tiles64 * 2 > sms || k_blocks < 8) return 1;
    long want = sms / tiles64;
    if (want > k_blocks / 4) want = k_blocks / 4;
    if (want > kMaxKSplits) want = kMaxKSplits;
    if (want < 2) return 1;
    const int per = (k_blocks + (int)want - 1) / (int)want;
    return (k_blocks + per - 1) / per;
}

}  // namespace nnis

// How many CTAs share a tile of the adding product of these sizes (1: no split of K),
// and the scratch that takes: `*floats` float32 and `*tiles` tickets.
NNIS_API int nnis_gemm_tc_splits(int M, int N, int K, int sm_count, long long* floats, int* tiles) {
    using namespace nnis;
    const int sms = sm_count > 0 ? sm_count : 148;
    const long m_tiles = (M + kBM - 1) / kBM;
    const long tiles128 = (long)((N + 127) / 128) * m_tiles;
    const long tiles64 = m_tiles * ((N + 63) / 64);
    const int splits = tiles128 >= sms ? 1 : gemm_k_splits(tiles64, K, sms);
    if (floats) *floats = splits > 1 ? tiles64 * splits * (long long)(kBM * 64) : 0;
    if (tiles) *tiles = splits > 1 ? (int)tiles64 : 0;
    return splits;
}

// Modes: 0 store bfloat16, 1 store float32, 2 add into float32, 3 gated
// (W = [gate rows; up rows], out [M, N / 2] = bf16(silu(gate) * up)), 4 QKV (bias,
// RoPE, q to out [M, nq * d], k and v into the paged cache; d must be 64 or 128).
// Refuses (NNIS_ERR_UNSUPPORTED): K not a multiple of 8, grids too large, a
// driver without tensor-map encoding; operands must be 16-byte aligned.
// `split_scratch` (`split_floats` float32) and `split_tickets` (`split_tiles` counters,
// zero before the first launch; the kernel leaves them zero) are optional: with them the
// adding mode cuts a long K among several CTAs per tile where tiles are few (see
// nnis_gemm_tc_splits).
NNIS_API int nnis_gemm_tc(const void* A, const void* W, const float* bias, void* C, int M, int N,
                          int K, int mode, const int* token_pos, const int* token_seq,
                          const int* page_table, int table_cols, const float* cos_t,
                          const float* sin_t, void* k_cache, void* v_cache, int nq, int nkv, int d,
                          int page_size, float* split_scratch, long long split_floats,
                          unsigned* split_tickets, int split_tiles, int sm_count, int* status, int pdl,
                          cudaStream_t stream) {
    using namespace nnis;
    if (M <= 0 || N <= 0 || K <= 0 || !A || !W || !C || mode < 0 || mode > 4) return NNIS_ERR_ARGUMENT;
    if (K % 8) return NNIS_ERR_UNSUPPORTED;
    if (((uintptr_t)A | (uintptr_t)W) % 16) return NNIS_ERR_ALIGNMENT;
    if (((uintptr_t)C % 16) != 0) return NNIS_ERR_ALIGNMENT;
    if ((M + kBM - 1) / kBM > 65535) return NNIS_ERR_UNSUPPORTED;
    GemmArgs g;
    g.bias = bias; g.out = C; g.M = M; g.N = N; g.K = K; g.status = status;
    g.token_pos = token_pos; g.token_seq = token_seq; g.page_table = page_table;
    g.table_cols = table_cols; g.cos_t = cos_t; g.sin_t = sin_t; g.k_cache = (bf16*)k_cache;
    g.v_cache = (bf16*)v_cache; g.nq = nq; g.nkv = nkv; g.d = d; g.page_size = page_size;
    g.k_splits = 1; g.split_scratch = nullptr; g.split_tickets = nullptr;
    static const char* const kNames[] = {"gemm store", "gemm store_f32", "gemm add_f32", "gemm gated", "gemm qkv"};
    g.trace = trace_slot(mode >= 0 && mode <= 4 ? kNames[mode] : "gemm");
    int sms = sm_count > 0 ? sm_count : 148;
    CUtensorMap ma, mw, mo;
    const long m_tiles = (M + kBM - 1) / kBM;
    // Two ring sizes per tile shape.  About 96 KB lets two CTAs share an SM, so that
    // one's epilogue runs under the other's products; when there are no more CTAs
    // than SMs a CTA takes about 192 KB instead, which keeps a microsecond of loads
    // in flight (a stage comes back about 1,000 cycles after its load is issued).
#define NNIS_GEMM_TC64(MODE, CTAS) \
    return (CTAS) <= sms ? launch_gemm_tc<64, 2, MODE, 4>(ma, mw, mo, g, pdl != 0, stream) \
                         : launch_gemm_tc<64, 2, MODE, 2>(ma, mw, mo, g, pdl != 0, stream)
#define NNIS_GEMM_TC128(BN, MODE, CTAS) \
    return (CTAS) <= sms ? launch_gemm_tc<BN, 3, MODE, 2>(ma, mw, mo, g, pdl != 0, stream) \
                         : launch_gemm_tc<BN, 3, MODE, 1>(ma, mw, mo, g, pdl != 0, stream)
    if (mode == GEMM_QKV) {
        if ((d != 64 && d != 128) || N != (nq + 2 * nkv) * d || !token_pos) return NNIS_ERR_UNSUPPORTED;
        if (nkv > 0 && (!token_seq || !page_table || !k_cache || !v_cache || page_size <= 0))
            return NNIS_ERR_ARGUMENT;
        if (!make_map(&ma, A, M, K, kBM) || !make_map(&mw, W, N, K, 128)) return NNIS_ERR_UNSUPPORTED;
        mo = ma;  // not used: this epilogue scatters rows into the cache
        g.out_by_tma = 0;
        NNIS_GEMM_TC128(128, GEMM_QKV, m_tiles * ((N + 127) / 128));
    }
    if (mode == GEMM_GATED) {
        if (N % 2) return NNIS_ERR_UNSUPPORTED;
        // wide outputs: 192 gate and 192 up columns per CTA, which has its SM alone
        // (384 columns of tensor memory, 64 KB a stage); products of N = 192 run at
        // the tensor cores' full rate, those of N = 64 at two thirds of it
        // (with enough fat tiles for half of the SMs; with fewer, as with one tile of rows in
        // a decode step of many sequences, three times as many narrow tiles pull the weights
        // from memory faster: 1.7B shape at 64 rows 28 -> 18 us)
        const bool fat = N / 2 > 128 && 2 * m_tiles * ((N / 2 + 191) / 192) >= sms;
        if (!make_map(&ma, A, M, K, kBM) || !make_map(&mw, W, N, K, fat ? 192 : 64)) return NNIS_ERR_UNSUPPORTED;
        g.out_by_tma = (N / 2) % 8 == 0 && make_map(&mo, C, M, N / 2, kBM);
        if (!g.out_by_tma) mo = ma;
        if (fat) return launch_gemm_tc<192, 3, GEMM_GATED, 1>(ma, mw, mo, g, pdl != 0, stream);
        NNIS_GEMM_TC128(64, GEMM_GATED, m_tiles * ((N / 2 + 63) / 64));
    }
    long tiles128 = (long)((N + 127) / 128) * m_tiles;
    bool wide = tiles128 >= sms;
    if (!make_map(&ma, A, M, K, kBM) || !make_map(&mw, W, N, K, wide ? 128 : 64))
        return NNIS_ERR_UNSUPPORTED;
    g.out_by_tma = mode == GEMM_STORE ? (N % 8 == 0 && make_map(&mo, C, M, N, kBM))
                                      : (N % 4 == 0 && make_map(&mo, C, M, N, kBM, 0, 4));
    if (!g.out_by_tma) mo = ma;
#define NNIS_GEMM_TC(MODE) \
    if (wide) NNIS_GEMM_TC128(128, MODE, tiles128); \
    NNIS_GEMM_TC64(MODE, m_tiles * ((N + 63) / 64))
    if (mode == GEMM_STORE) { NNIS_GEMM_TC(GEMM_STORE); }
    if (mode == GEMM_STORE_F32) { NNIS_GEMM_TC(GEMM_STORE_F32); }
    const long tiles64 = m_tiles * ((N + 63) / 64);
    const int splits = wide ? 1 : gemm_k_splits(tiles64, K, sms);
    if (splits > 1 && split_scratch && split_tickets && tiles64 <= split_tiles &&
        tiles64 * splits * (long long)(kBM * 64) <= split_floats) {
        g.k_splits = splits; g.split_scratch = split_scratch; g.split_tickets = split_tickets;
        return launch_gemm_tc<64, 2, GEMM_ADD_F32, 4, true>(ma, mw, mo, g, pdl != 0, stream);
    }
    NNIS_GEMM_TC(GEMM_ADD_F32);
#undef NNIS_GEMM_TC64
#undef NNIS_GEMM_TC128
#undef NNIS_GEMM_TC
}
