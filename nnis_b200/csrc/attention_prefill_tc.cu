// Prompt attention over the paged bfloat16 cache on the fifth-generation tensor
// cores, for head size 64: packed query tokens of several sequences, each query
// over the keys of its own sequence up to its own position (and within the
// window, if there is one).
//
// One CTA owns 128 consecutive query tokens of one sequence, one query head and a
// range of that tile's pages (all of them, or one of several chunks when the host
// cuts long tiles so that there are CTAs enough for every SM and the late tiles of
// a long prompt do not run alone at the end).  Its eleven warps have fixed roles:
//   warp 0   one lane issues TMA loads: the Q tile [128, 64] once, then a page of
//            K and of V [64 keys, 64] per step of the loop into a ring of stages;
//   warp 1   allocates tensor memory; one lane issues, per page,
//            S[128, 64 keys] = Q . K^T        (tcgen05.mma, K-major operands)
//            as far ahead as the two buffers of S allow;
//   warp 2   one lane issues, per page,
//            O[128, 64]     += P . V          (P from shared memory, K-major;
//                                              V as loaded, i.e. MN-major)
//            (issuing a product and its barrier traffic costs one thread several
//            hundred cycles a page, so each product has a thread of its own);
//   warps 3-10 softmax, two warps per quarter of the rows: a thread has one query
//            row and one half of each page's keys; it reads its 32 scores from
//            tensor memory, masks them, keeps a maximum and a sum of its own
//            (float32, exp2), and writes P (bfloat16) into shared memory in the
//            128-byte-swizzled K-major layout the second product reads.  The halves
//            have accumulators O of their own (the second product's first two
//            K steps go to one, the last two to the other) and are merged at the end.
// S and P are double-buffered.  O stays in tensor memory for the whole tile: the
// maximum that P is taken against is only raised when a page's maximum exceeds it
// by more than 8 (a factor 256, harmless in float32 and bfloat16); then the warp
// waits for the products so far, multiplies its rows of O by exp2(old - new) in
// tensor memory and goes on.  Sum and output are relative to the same maximum, so
// the result is the exact softmax.
// A CTA with all pages of its tile writes bfloat16 output rows; a chunk writes its
// unnormalised rows, maxima and sums (float32) to scratch, takes a ticket, and the
// chunk that arrives last merges the chunks of the tile.
// The host lists the units (sequence, first query, chunk) because sequences have
// unequal lengths.  Every wait is bounded; a wait that runs out raises an abort flag that
// every role sees, all warps still meet at the end and tensor memory is freed.
// NNIS has a batched causal kernel on CUDA cores (crates/nnis-kernels/src/attention.rs:46-150).
#include <float.h>

#include "tcgen05_helpers.cuh"

namespace nnis {

constexpr int kTcRows = 128;     // queries per CTA
constexpr int kTcD = 64;         // head size
constexpr int kTcPage = 64;      // keys per page
constexpr int kTcStages = 3;     // K/V pages in flight
constexpr int kTcThreads = 352;  // loader, two issuers, eight softmax warps
constexpr float kTcLog2e = 1.4426950408889634f;
constexpr int kTcPartial = kTcD + 2;  // floats per row of a chunk's result: O, maximum, sum
constexpr float kTcRaise = 8.0f;  // log2 of how far a page's maximum may exceed the one in use

// V tile as loaded ([64 keys, 64 d], rows of 128 bytes, 128-byte swizzle) read as
// the MN-major B operand of O += P . V: 8-key groups are 1024 bytes apart.
__device__ __forceinline__ uint64_t smem_desc_mn128(uint32_t smem_byte_addr) {
    uint64_t desc = 0;
    desc |= (uint64_t)((smem_byte_addr >> 4) & 0x3FFF);
    desc |= (uint64_t)1 << 16;              // leading byte offset: one 64-wide chunk only, unused
    desc |= (uint64_t)(1024 >> 4) << 32;    // stride byte offset between groups of 8 keys
    desc |= (uint64_t)1 << 46;              // descriptor version of sm_100
    desc |= (uint64_t)2 << 61;              // SWIZZLE_128B
    return desc;
}

__device__ __forceinline__ float max3(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}

// 2^x for x <= 0 or so; -inf gives 0, denormal results are flushed
__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// Wait of a thread that has nothing else to do (the loader and the two issuers):
// it may stay suspended for up to two microseconds per try, so that its polling
// does not take issue slots from the softmax warp on the same scheduler.  False
// after `limit` tries (a quarter of a second).
__device__ __forceinline__ bool mbar_wait_idle(uint64_t* bar, uint32_t parity, uint32_t limit = 1u << 17) {
    const uint32_t addr = smem_addr(bar);
    for (uint32_t i = 0; i < limit; ++i) {
        uint32_t done;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(done)
            : "r"(addr), "r"(parity), "r"(2000u)
            : "memory");
        if (done) return true;
    }
    return false;
}

// Every lane polls (one lane polling for the others and handing the answer on by
// a shuffle measured slower); the vote makes the answer the warp's.
__device__ __forceinline__ bool warp_wait(uint64_t* bar, uint32_t parity, int lane) {
    (void)lane;
    return __all_sync(0xffffffffu, mbar_wait(bar, parity));
}

__device__ __forceinline__ void fence_async_smem() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

__device__ __forceinline__ void tmem_store32(uint32_t taddr, const uint32_t (&v)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
        "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
        ::"r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]),
          "r"(v[7]), "r"(v[8]), "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]),
          "r"(v[15]), "r"(v[16]), "r"(v[17]), "r"(v[18]), "r"(v[19]), "r"(v[20]), "r"(v[21]),
          "r"(v[22]), "r"(v[23]), "r"(v[24]), "r"(v[25]), "r"(v[26]), "r"(v[27]), "r"(v[28]),
          "r"(v[29]), "r"(v[30]), "r"(v[31])
        : "memory");
    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void tmem_load16(uint32_t taddr, uint32_t (&v)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]),
          "=r"(v[7]), "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]),
          "=r"(v[14]), "=r"(v[15])
        : "r"(taddr)
        : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_store16(uint32_t taddr, const uint32_t (&v)[16]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
        ::"r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]),
          "r"(v[7]), "r"(v[8]), "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]),
          "r"(v[15])
        : "memory");
    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}

__global__ void __launch_bounds__(kTcThreads, 2)
attn_prefill_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                       const __grid_constant__ CUtensorMap map_v, const int* __restrict__ units,
                       const int* __restrict__ seq_first_row, const int* __restrict__ seq_start,
                       const int* __restrict__ seq_count, const int* __restrict__ page_table,
                       int table_cols, bf16* __restrict__ out, float* __restrict__ partial,
                       unsigned* __restrict__ tickets, int nq, int nkv, int window, float scale,
                       int* __restrict__ status, unsigned long long* trace) {
    trace_mark(trace, 0);
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    unsigned char* base = reinterpret_cast<unsigned char*>(
        (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    constexpr uint32_t kBytesQ = kTcRows * kTcD * 2, kBytesKV = kTcPage * kTcD * 2;
    unsigned char* q_s = base;                                   // [128, 64] swizzled
    unsigned char* p_s = q_s + kBytesQ;                          // 2 x [128, 64 keys] swizzled
    unsigned char* k_s = p_s + 2 * kBytesQ;                      // stages x [64, 64]
    unsigned char* v_s = k_s + kTcStages * kBytesKV;
    __shared__ __align__(8) uint64_t q_full, kv_full[kTcStages], kv_empty[kTcStages];
    __shared__ __align__(8) uint64_t s_full[2], s_free[2], p_ready[2], p_free[2], o_full, halves_met;
    __shared__ float half_m[2][kTcRows], half_l[2][kTcRows];  // each half's maximum and sum, for the other
    __shared__ __align__(8) uint64_t chunk_written, last_known;
    __shared__ int is_last_chunk;
    __shared__ uint32_t tmem_base_s;
    __shared__ volatile int abort_flag;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // the host lists the units with the most pages first
    const int4 unit = reinterpret_cast<const int4*>(units)[blockIdx.x];
    const int seq = unit.x, q0 = unit.y, chunk = unit.z & 0xffff, n_chunks = unit.z >> 16;
    const int hq = blockIdx.y, hk = hq / (nq / nkv);
    const int count = seq_count[seq], start = seq_start[seq];
    const int row_base = seq_first_row[seq] + q0;
    const int rows = min(kTcRows, count - q0);
    const int pos0 = start + q0;
    const int hi = pos0 + rows;
    const int lo = window > 0 ? max(0, pos0 - window + 1) : 0;
    const int tile_first = lo / kTcPage, tile_pages = (hi - 1) / kTcPage - tile_first + 1;
    const int per_chunk = (tile_pages + n_chunks - 1) / n_chunks;
    const int first_page = tile_first + chunk * per_chunk;
    const int n_pages = min(per_chunk, tile_pages - chunk * per_chunk);  // >= 1 by the host's plan
    const int* table = page_table + (size_t)seq * table_cols;

    if (threadIdx.x == 64) {
        prefetch_tensormap(&map_q);
        prefetch_tensormap(&map_k);
        prefetch_tensormap(&map_v);
    }
    if (threadIdx.x == 0) {
        mbar_init(&q_full, 1);
        for (int s = 0; s < kTcStages; ++s) {
            mbar_init(&kv_full[s], 1);
            mbar_init(&kv_empty[s], 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&s_full[b], 2);    // S(i) is there, and P's buffer of page i is free again
            mbar_init(&s_free[b], 8);    // one arrival per softmax warp
            mbar_init(&p_ready[b], 8);
            mbar_init(&p_free[b], 1);
        }
        mbar_init(&o_full, 1);
        mbar_init(&halves_met, 8);
        mbar_init(&chunk_written, 8);
        mbar_init(&last_known, 1);
        abort_flag = 0;
        mbar_fence_init();
    }
    if (warp == 1) tmem_alloc(&tmem_base_s, 256);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    // S: two buffers of 64 columns; O: one accumulator of 64 columns per half of a page's keys
    const uint32_t tmem_s = tmem_base_s, tmem_o = tmem_base_s + 128;
    // launched as a programmatic dependent: the queries, and this step's keys and
    // values, come from the kernel before this one; the set-up above ran under it
    pdl_wait();
    pdl_launch_dependents();
    trace_mark(trace, 2);
    trace_mark(trace, 3);

    if (warp == 0) {
        if (lane == 0) {
            mbar_expect_tx(&q_full, kBytesQ);
            tma_load_2d(q_s, &map_q, hq * kTcD, row_base, &q_full);
            for (int i = 0; i < n_pages; ++i) {
                int s = i % kTcStages;
                if (i >= kTcStages && !mbar_wait_idle(&kv_empty[s], (uint32_t)(i / kTcStages - 1) & 1u)) {
                    abort_flag = 1;
                    break;
                }
                if (abort_flag) break;
                int page = table[first_page + i];
                int row = (page * nkv + hk) * kTcPage;
                mbar_expect_tx(&kv_full[s], 2 * kBytesKV);
                tma_load_2d(k_s + (size_t)s * kBytesKV, &map_k, 0, row, &kv_full[s]);
                tma_load_2d(v_s + (size_t)s * kBytesKV, &map_v, 0, row, &kv_full[s]);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            // S(i) = Q K(i)^T, both operands K-major (d contiguous), as far ahead as
            // the two buffers of S and the ring of pages allow
            constexpr uint32_t idesc_s = instr_desc(kTcRows, kTcPage);
            const uint64_t desc_q = smem_desc_k128(smem_addr(q_s)), desc_k0 = smem_desc_k128(smem_addr(k_s));
            bool ok = mbar_wait_idle(&q_full, 0);
            for (int i = 0; ok && i < n_pages; ++i) {
                int s = i % kTcStages, b = i & 1;
                ok = mbar_wait_idle(&kv_full[s], (uint32_t)(i / kTcStages) & 1u) && !abort_flag;
                if (ok && i >= 2) ok = mbar_wait_idle(&s_free[b], (uint32_t)((i >> 1) - 1) & 1u);
                if (!ok) break;
                tc_fence_after();
                const uint64_t desc_k = desc_advance(desc_k0, (uint32_t)s * kBytesKV);
#pragma unroll
                for (int k = 0; k < kTcD / 16; ++k)
                    tc_mma(tmem_s + b * 64, desc_advance(desc_q, k * 32), desc_advance(desc_k, k * 32),
                           idesc_s, k != 0);
                tc_commit(&s_full[b]);
            }
            if (!ok) abort_flag = 1;
        }
    } else if (warp == 2) {
        if (lane == 0) {
            // O += P(i) V(i): P K-major (keys contiguous), V MN-major (d contiguous,
            // keys across rows).  S(i) was complete before P(i) could be made, so the
            // commit after this product also frees the page's K.
            constexpr uint32_t idesc_o = instr_desc(kTcRows, kTcD) | (1u << 16);
            const uint64_t desc_p0 = smem_desc_k128(smem_addr(p_s)), desc_v0 = smem_desc_mn128(smem_addr(v_s));
            bool ok = true;
            // both buffers of P are free for the first two pages
            mbar_arrive(&s_full[0]);
            mbar_arrive(&s_full[1]);
            for (int i = 0; i < n_pages; ++i) {
                int s = i % kTcStages, b = i & 1;
                ok = mbar_wait_idle(&p_ready[b], (uint32_t)(i >> 1) & 1u) && !abort_flag;
                if (!ok) break;
                tc_fence_after();
                const uint64_t desc_p = desc_advance(desc_p0, (uint32_t)b * kBytesQ);
                const uint64_t desc_v = desc_advance(desc_v0, (uint32_t)s * kBytesKV);
#pragma unroll
                for (int k = 0; k < kTcPage / 16; ++k)  // keys 0-31 into the first O, 32-63 into the second
                    tc_mma(tmem_o + (k >> 1) * 64, desc_advance(desc_p, k * 32), desc_advance(desc_v, k * 2048),
                           idesc_o, (i | (k & 1)) != 0);
                tc_commit(&p_free[b]);
                tc_commit(&s_full[b]);  // counts for page i + 2, which writes this buffer of P
                tc_commit(&kv_empty[s]);
            }
            if (ok) tc_commit(&o_full);
            else abort_flag = 1;
        }
    } else {
        // Softmax.  Two warps share each quarter of the rows (a warp alone on its
        // scheduler hides no latency); a thread has one row and one half of every
        // page's keys, with a running maximum, sum and accumulator O of its own for
        // that half, so the halves never wait for each other until the end.
        const int quarter = warp & 3, half = (warp - 3) >> 2;
        const int row = quarter * 32 + lane;
        const uint32_t lane_base = (uint32_t)(quarter * 32) << 16;
        const uint32_t my_o = tmem_o + half * 64 + lane_base;
        const int pos = pos0 + row;
        const int lo_row = window > 0 ? pos - window + 1 : 0;
        // the keys every row of this warp sees whole: no masking on such pages
        const int warp_pos_min = pos0 + quarter * 32;
        const int warp_lo_max = window > 0 ? warp_pos_min + 31 - window + 1 : 0;
        const float sc = scale * kTcLog2e;
        float m_run = -INFINITY, l_run = 0.f;  // maximum in use (scaled, log2 units) and sum against it
        bool ok = true;
        for (int i = 0; i < n_pages; ++i) {
            const int b = i & 1;
            ok = warp_wait(&s_full[b], (uint32_t)(i >> 1) & 1u, lane) && !abort_flag;
            if (!ok) break;
            tc_fence_after();
            uint32_t sv[32];
            tmem_load32(tmem_s + b * 64 + half * 32 + lane_base, sv);
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&s_free[b]);  // this buffer may take the page after next
            const int t0 = (first_page + i) * kTcPage + half * 32;
            if (t0 + 31 > warp_pos_min || t0 < warp_lo_max) {
#pragma unroll
                for (int c = 0; c < 32; ++c)
                    if (t0 + c > pos || t0 + c < lo_row) sv[c] = 0xff800000u;  // -inf
            }
            float mx[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
            for (int c = 0; c < 32; c += 8)  // (the maximum of three in one instruction)
#pragma unroll
                for (int e = 0; e < 4; ++e)
                    mx[e] = max3(mx[e], __uint_as_float(sv[c + 2 * e]), __uint_as_float(sv[c + 2 * e + 1]));
            const float m_page = fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3])) * sc;
            const float m_new = fmaxf(m_run, m_page);
            const bool raise = m_run != -INFINITY && m_new > m_run + kTcRaise;
            if (m_run == -INFINITY) m_run = m_new;  // nothing summed yet: this row of O is zero
            if (i > 0 && __any_sync(0xffffffffu, raise)) {
                // every product so far has to be in O before it is rescaled
                ok = warp_wait(&p_free[(i - 1) & 1], (uint32_t)((i - 1) >> 1) & 1u, lane);
                if (!ok) break;
                tc_fence_after();
                const float alpha = m_run == -INFINITY ? 1.f : exp2f(m_run - m_new);
#pragma unroll 1
                for (int h = 0; h < 4; ++h) {
                    uint32_t ov[16];
                    tmem_load16(my_o + h * 16, ov);
#pragma unroll
                    for (int c = 0; c < 16; ++c) ov[c] = __float_as_uint(__uint_as_float(ov[c]) * alpha);
                    tmem_store16(my_o + h * 16, ov);
                }
                l_run *= alpha;
                m_run = m_new;
            }
            const float neg_base = m_run == -INFINITY ? 0.f : -m_run;
            // (the product that read this buffer of P two pages ago is over: s_full said so)
            unsigned char* p_row = p_s + (size_t)b * kBytesQ + (size_t)row * 128;
            float ps[4] = {0.f, 0.f, 0.f, 0.f};
            // P row: 8 chunks of 8 keys, four of them this thread's; chunk j lands at
            // 16-byte slot j ^ (row % 8)
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                uint32_t w[4];
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    int c = j * 8 + e * 2;
                    float p0 = ex2(fmaf(__uint_as_float(sv[c]), sc, neg_base));
                    float p1 = ex2(fmaf(__uint_as_float(sv[c + 1]), sc, neg_base));
                    ps[e] += p0 + p1;
                    __nv_bfloat162 pk = __floats2bfloat162_rn(p0, p1);
                    w[e] = *reinterpret_cast<uint32_t*>(&pk);
                }
                *reinterpret_cast<uint4*>(p_row + (((half * 4 + j) ^ (row & 7)) << 4)) =
                    make_uint4(w[0], w[1], w[2], w[3]);
            }
            l_run += (ps[0] + ps[1]) + (ps[2] + ps[3]);
            fence_async_smem();  // the tensor core reads P through the async proxy
            tc_fence_before();   // and a rescaled O through tensor memory
            __syncwarp();
            if (lane == 0) mbar_arrive(&p_ready[b]);
        }
        // the halves meet: each needs the other's maximum and sum
        half_m[half][row] = m_run;
        half_l[half][row] = l_run;
        __syncwarp();
        if (ok && lane == 0) mbar_arrive(&halves_met);
        ok = ok && warp_wait(&halves_met, 0, lane) && warp_wait(&o_full, 0, lane) && !abort_flag;
        if (!ok) {
            abort_flag = 1;
        } else {
            tc_fence_after();
            // this thread finishes 32 of the row's 64 output columns from both accumulators
            const float m_a = half_m[0][row], m_b = half_m[1][row];
            const float m_all = fmaxf(m_a, m_b);
            const float w_a = m_a == -INFINITY ? 0.f : exp2f(m_a - m_all);
            const float w_b = m_b == -INFINITY ? 0.f : exp2f(m_b - m_all);
            const float l_all = w_a * half_l[0][row] + w_b * half_l[1][row];
            uint32_t oa[32], ob[32];
            tmem_load32_issue(tmem_o + lane_base + half * 32, oa);
            tmem_load32_issue(tmem_o + 64 + lane_base + half * 32, ob);
            tmem_load_wait();
            tc_fence_before();
            if (n_chunks == 1) {
                const float inv = l_all > 0.f ? 1.0f / l_all : 0.f;
                const float f_a = w_a * inv, f_b = w_b * inv;
                if (row < rows) {
                    bf16* dst = out + (size_t)(row_base + row) * nq * kTcD + (size_t)hq * kTcD + half * 32;
#pragma unroll
                    for (int c = 0; c < 32; c += 8) {
                        uint32_t w[4];
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            float x0 = f_a * __uint_as_float(oa[c + 2 * e]) + f_b * __uint_as_float(ob[c + 2 * e]);
                            float x1 = f_a * __uint_as_float(oa[c + 2 * e + 1]) + f_b * __uint_as_float(ob[c + 2 * e + 1]);
                            __nv_bfloat162 a = __floats2bfloat162_rn(x0, x1);
                            w[e] = *reinterpret_cast<uint32_t*>(&a);
                        }
                        *reinterpret_cast<uint4*>(dst + c) = make_uint4(w[0], w[1], w[2], w[3]);
                    }
                }
            } else {
                // One of several chunks of this tile's pages: its unnormalised rows,
                // maxima and sums go to scratch, [kTcPartial][128 rows] float32 per
                // (slot, head), column-major so that a warp's 32 rows are one 128-byte
                // line; the chunk that finds all others written merges them, in the
                // order of the chunks whichever came last.
                const size_t per_chunk_floats = (size_t)nq * (kTcPartial * kTcRows);
                float* tile_partial = partial + ((size_t)unit.w * nq + hq) * (kTcPartial * kTcRows) + row;
                float* dst = tile_partial + (size_t)chunk * per_chunk_floats;
#pragma unroll
                for (int c = 0; c < 32; ++c)
                    dst[(size_t)(half * 32 + c) * kTcRows] =
                        w_a * __uint_as_float(oa[c]) + w_b * __uint_as_float(ob[c]);
                if (half == 0) {
                    dst[(size_t)kTcD * kTcRows] = m_all;
                    dst[(size_t)(kTcD + 1) * kTcRows] = l_all;
                }
                __threadfence();
                __syncwarp();
                if (lane == 0) mbar_arrive(&chunk_written);
                if (warp == 3 && lane == 0) {
                    if (mbar_wait(&chunk_written, 0)) {
                        unsigned* ticket = tickets + (size_t)unit.w * nq + hq;
                        const bool last = atomicAdd(ticket, 1u) == (unsigned)n_chunks - 1u;
                        if (last) *ticket = 0u;  // the next launch finds it zero
                        is_last_chunk = last ? 1 : 0;
                    } else {
                        is_last_chunk = 0;
                        abort_flag = 1;
                    }
                    mbar_arrive(&last_known);
                }
                if (warp_wait(&last_known, 0, lane) && is_last_chunk && !abort_flag) {
                    __threadfence();
                    float m_tile = -INFINITY;
                    for (int c = 0; c < n_chunks; ++c)
                        m_tile = fmaxf(m_tile, __ldcg(tile_partial + (size_t)c * per_chunk_floats + (size_t)kTcD * kTcRows));
                    float acc[32];
#pragma unroll
                    for (int j = 0; j < 32; ++j) acc[j] = 0.f;
                    float l_tile = 0.f;
                    for (int c = 0; c < n_chunks; ++c) {
                        const float* src = tile_partial + (size_t)c * per_chunk_floats;
                        const float mc = __ldcg(src + (size_t)kTcD * kTcRows);
                        if (mc == -INFINITY) continue;  // no key of this chunk was visible to the row
                        const float wc = exp2f(mc - m_tile);
                        l_tile = fmaf(wc, __ldcg(src + (size_t)(kTcD + 1) * kTcRows), l_tile);
#pragma unroll
                        for (int j = 0; j < 32; ++j)
                            acc[j] = fmaf(wc, __ldcg(src + (size_t)(half * 32 + j) * kTcRows), acc[j]);
                    }
                    const float inv = l_tile > 0.f ? 1.0f / l_tile : 0.f;
                    if (row < rows) {
                        bf16* o_dst = out + (size_t)(row_base + row) * nq * kTcD + (size_t)hq * kTcD + half * 32;
#pragma unroll
                        for (int j = 0; j < 32; j += 8) {
                            uint32_t w[4];
#pragma unroll
                            for (int e = 0; e < 4; ++e) {
                                __nv_bfloat162 a = __floats2bfloat162_rn(acc[j + 2 * e] * inv, acc[j + 2 * e + 1] * inv);
                                w[e] = *reinterpret_cast<uint32_t*>(&a);
                            }
                            *reinterpret_cast<uint4*>(o_dst + j) = make_uint4(w[0], w[1], w[2], w[3]);
                        }
                    }
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base_s, 256);
    }
    if (threadIdx.x == 0 && abort_flag && status) atomicExch(status, 4);
    trace_mark(trace, 1);
}

}  // namespace nnis

// `units`: int32 [n_units, 4] = (sequence of the batch, first query of the tile
// within this step's tokens of that sequence, chunk | chunks << 16, first scratch
// slot of the tile), 128 queries per tile, the pages of a tile cut into `chunks`
// equal ranges (the last may be shorter, none empty).  `partial`: float32
// [slots, nq, 66, 128] scratch and `tickets`: [slots, nq] counters, zero before the
// first launch and left zero, both only when tiles were cut.  Per sequence
// `seq_first_row`, `seq_start`, `seq_count` as for nnis_attention_prefill_mma.
// q: [n_tokens, nq * 64] bfloat16 with rows `q_stride` elements apart (a multiple
// of 8).  Takes head size 64 with 64-key pages; else NNIS_ERR_UNSUPPORTED.  `pdl`:
// launch as a programmatic dependent of the kernel before it on the stream.
NNIS_API int nnis_attention_prefill_tc(const void* q, int q_stride, int n_tokens, const void* k_cache,
                                       const void* v_cache, long long cache_rows, const int* units,
                                       int n_units, float* partial, unsigned* tickets,
                                       const int* seq_first_row, const int* seq_start,
                                       const int* seq_count, const int* page_table, int table_cols,
                                       void* out, int nq, int nkv, int d, int page_size, int window,
                                       float scale, int* status, int pdl, cudaStream_t stream) {
    using namespace nnis;
    if (n_units <= 0 || n_tokens <= 0 || nq <= 0 || nkv <= 0 || nq % nkv || table_cols <= 0 ||
        window < 0 || !units || cache_rows <= 0 || q_stride < nq * d || !(scale > 0.f) ||
        ((partial == nullptr) != (tickets == nullptr)))
        return NNIS_ERR_ARGUMENT;
    if (d != kTcD || page_size != kTcPage || nq > 65535 || q_stride % 8) return NNIS_ERR_UNSUPPORTED;
    if (((uintptr_t)q | (uintptr_t)k_cache | (uintptr_t)v_cache | (uintptr_t)out | (uintptr_t)units |
         (uintptr_t)partial) % 16)
        return NNIS_ERR_ALIGNMENT;
    CUtensorMap mq, mk, mv;
    if (!make_map(&mq, q, n_tokens, nq * kTcD, kTcRows, q_stride) ||
        !make_map(&mk, k_cache, cache_rows, kTcD, kTcPage) || !make_map(&mv, v_cache, cache_rows, kTcD, kTcPage))
        return NNIS_ERR_UNSUPPORTED;
    size_t smem = 3 * (size_t)kTcRows * kTcD * 2 + 2 * (size_t)kTcStages * kTcPage * kTcD * 2 + 1024;
    cudaError_t e = cudaFuncSetAttribute(attn_prefill_tc_kernel,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(n_units, nq);
    cfg.blockDim = dim3(kTcThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 1 : 0;
    e = cudaLaunchKernelEx(&cfg, attn_prefill_tc_kernel, mq, mk, mv, units, seq_first_row, seq_start,
                           seq_count, page_table, table_cols, (bf16*)out, partial, tickets, nq, nkv,
                           window, scale, status, trace_slot("attention prompt (tcgen05)"));
    return e == cudaSuccess ? NNIS_OK : (int)e;
}
