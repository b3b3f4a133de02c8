// Decode attention over the paged cache in bfloat16: one query token per
// sequence against its whole context, bound by the bytes of K and V.
//
// One CTA owns (kv head, up to four of its query heads, sequence, slice of the
// key range).  K and V rows are read once with 16-byte loads and serve all the
// query heads of the group.  LPK lanes share one key (each holds 8 of its
// head_dim elements), so a warp covers 32 / LPK keys per pass; every such lane
// group runs its own online softmax in float32 over the keys it meets, and the
// groups, warps and slices are merged afterwards with the usual (max, sum,
// output) rule in a fixed order.  Slices write float32 partial records that the
// merge kernel of attention_generic.cu turns into the output.
//
// Sizes: head_dim any multiple of 16 up to 256, any heads / kv_heads ratio, an
// optional window.  NNIS: crates/nnis-model/src/kernels.rs:66-125 and its
// 64-lane variant crates/nnis-model/src/cached_attention_candidate.rs:16-86.
#include <float.h>

#include "async_copy.cuh"
#include "common.cuh"

namespace nnis {

__device__ __forceinline__ void unpack8(const uint4& raw, float* f) {
    f[0] = __uint_as_float(raw.x << 16);
    f[1] = __uint_as_float(raw.x & 0xffff0000u);
    f[2] = __uint_as_float(raw.y << 16);
    f[3] = __uint_as_float(raw.y & 0xffff0000u);
    f[4] = __uint_as_float(raw.z << 16);
    f[5] = __uint_as_float(raw.z & 0xffff0000u);
    f[6] = __uint_as_float(raw.w << 16);
    f[7] = __uint_as_float(raw.w & 0xffff0000u);
}

// Merge stream b into stream a: (m, l, acc[8]) per head.
template <int GT>
__device__ __forceinline__ void merge_streams(float* m, float* l, float (*acc)[8], const float* mb,
                                              const float* lb, const float (*accb)[8]) {
#pragma unroll
    for (int g = 0; g < GT; ++g) {
        float mn = fmaxf(m[g], mb[g]);
        float sa = l[g] > 0.f ? __expf(m[g] - mn) : 0.f;
        float sb = lb[g] > 0.f ? __expf(mb[g] - mn) : 0.f;
        l[g] = l[g] * sa + lb[g] * sb;
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[g][i] = acc[g][i] * sa + accb[g][i] * sb;
        m[g] = mn;
    }
}

constexpr int kDecodeWarps = 4;

// K and V of one page and kv head are contiguous in the cache
// ([pages, kv_heads, page_size, d]), so a page comes in with two bulk copies.
// `stages` pages are in flight per CTA; dynamic shared memory holds
// stages x (K tile, V tile) and one mbarrier per stage.
template <int LPK, int GT>
__global__ void __launch_bounds__(kDecodeWarps * 32)
attn_decode_kernel(const bf16* __restrict__ q, int q_stride, const bf16* __restrict__ k_cache,
                   const bf16* __restrict__ v_cache, const int* __restrict__ token_pos,
                   const int* __restrict__ token_seq, const int* __restrict__ page_table,
                   int table_cols, bf16* __restrict__ out, float* __restrict__ partial, int nq,
                   int nkv, int d, int page_size, int window, float scale, int n_splits,
                   int head_tiles, int stages, int* __restrict__ status) {
    constexpr int KPW = 32 / LPK;  // keys per warp and pass
    extern __shared__ __align__(128) unsigned char smem_raw[];
    __shared__ float sm_m[kDecodeWarps][GT], sm_l[kDecodeWarps][GT];
    __shared__ float sm_acc[kDecodeWarps][GT][LPK * 8];
    __shared__ int sm_failed;

    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int sub = lane % LPK, grp = lane / LPK;
    const int hk = blockIdx.x / head_tiles, tile = blockIdx.x % head_tiles;
    const int G = nq / nkv;
    const int g0 = tile * GT;
    const int gcount = min(GT, G - g0);
    const int n = blockIdx.y, split = blockIdx.z;
    const bool active = sub * 8 < d;
    const size_t tile_elems = (size_t)page_size * d;
    bf16* tiles = reinterpret_cast<bf16*>(smem_raw);
    uint64_t* bars = reinterpret_cast<uint64_t*>(tiles + (size_t)stages * 2 * tile_elems);

    float m[GT], l[GT], acc[GT][8];
#pragma unroll
    for (int g = 0; g < GT; ++g) {
        m[g] = -FLT_MAX;
        l[g] = 0.f;
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[g][i] = 0.f;
    }

    if (threadIdx.x == 0) {
        for (int s = 0; s < stages; ++s) mbar_init(bars + s, 1);
        mbar_fence_init();
        sm_failed = 0;
    }
    // the position, the page table and this token's own key and value come from
    // kernels before this one
    pdl_wait();
    const int pos = token_pos[n];
    __syncthreads();

    if (pos >= 0) {
        const int lo = window > 0 ? max(0, pos - window + 1) : 0;
        const int hi = pos + 1;
        const int first_page = lo / page_size, last_page = (hi - 1) / page_size;
        const int per = (last_page - first_page + n_splits) / n_splits;
        const int p0 = first_page + split * per;
        const int count = max(0, min(last_page + 1, p0 + per) - p0);
        const int* table = page_table + (size_t)token_seq[n] * table_cols;
        const uint32_t tile_bytes = (uint32_t)(tile_elems * sizeof(bf16));

        auto issue = [&](int it) {  // thread 0 only
            int page = table[p0 + it];
            size_t src = (size_t)(page * nkv + hk) * tile_elems;
            uint64_t* bar = bars + (it % stages);
            bf16* dst = tiles + (size_t)(it % stages) * 2 * tile_elems;
            mbar_expect_tx(bar, 2u * tile_bytes);
            bulk_load(dst, k_cache + src, tile_bytes, bar);
            bulk_load(dst + tile_elems, v_cache + src, tile_bytes, bar);
        };
        if (threadIdx.x == 0)
            for (int it = 0; it < min(stages, count); ++it) issue(it);
        pdl_launch_dependents();

        float qf[GT][8];
#pragma unroll
        for (int g = 0; g < GT; ++g) {
#pragma unroll
            for (int i = 0; i < 8; ++i) qf[g][i] = 0.f;
            if (g < gcount && active) {
                const bf16* qp = q + (size_t)n * q_stride + (size_t)(hk * G + g0 + g) * d + sub * 8;
                uint4 raw = *reinterpret_cast<const uint4*>(qp);
                unpack8(raw, qf[g]);
#pragma unroll
                for (int i = 0; i < 8; ++i) qf[g][i] *= scale;
            }
        }
        for (int it = 0; it < count; ++it) {
            // a wait that runs out is recorded and acted on after the barrier below,
            // where every thread sees it, so that no thread leaves the loop alone
            if (!mbar_wait(bars + (it % stages), (uint32_t)(it / stages) & 1u)) sm_failed = 1;
            const bf16* kt = tiles + (size_t)(it % stages) * 2 * tile_elems;
            const bf16* vt = kt + tile_elems;
            const int t0 = (p0 + it) * page_size;
            // the same number of passes for every lane, so the shuffles below meet
            for (int kb = warp * KPW; kb < page_size; kb += kDecodeWarps * KPW) {
                const int key = kb + grp;
                const int t = t0 + key;
                const bool valid = key < page_size && t >= lo && t < hi;
                uint4 kr = make_uint4(0, 0, 0, 0), vr = make_uint4(0, 0, 0, 0);
                if (valid && active) {
                    kr = *reinterpret_cast<const uint4*>(kt + (size_t)key * d + sub * 8);
                    vr = *reinterpret_cast<const uint4*>(vt + (size_t)key * d + sub * 8);
                }
                float kf[8], vf[8];
                unpack8(kr, kf);
                unpack8(vr, vf);
#pragma unroll
                for (int g = 0; g < GT; ++g) {
                    float s = 0.f;
#pragma unroll
                    for (int i = 0; i < 8; ++i) s = fmaf(qf[g][i], kf[i], s);
#pragma unroll
                    for (int o = LPK / 2; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
                    if (valid) {
                        float mn = fmaxf(m[g], s);
                        float alpha = __expf(m[g] - mn);  // m = -FLT_MAX at first: exp(-huge) = 0
                        float p = __expf(s - mn);
                        l[g] = l[g] * alpha + p;
#pragma unroll
                        for (int i = 0; i < 8; ++i) acc[g][i] = fmaf(p, vf[i], acc[g][i] * alpha);
                        m[g] = mn;
                    }
                }
            }
            __syncthreads();  // every warp is done with this stage
            if (sm_failed) break;
            if (threadIdx.x == 0 && it + stages < count) issue(it + stages);
        }
        if (sm_failed && threadIdx.x == 0 && status) atomicExch(status, 2);
        // the key groups of a warp, in a fixed butterfly order
#pragma unroll
        for (int off = LPK; off < 32; off <<= 1) {
            float mb[GT], lb[GT], accb[GT][8];
#pragma unroll
            for (int g = 0; g < GT; ++g) {
                mb[g] = __shfl_xor_sync(0xffffffffu, m[g], off);
                lb[g] = __shfl_xor_sync(0xffffffffu, l[g], off);
#pragma unroll
                for (int i = 0; i < 8; ++i) accb[g][i] = __shfl_xor_sync(0xffffffffu, acc[g][i], off);
            }
            merge_streams<GT>(m, l, acc, mb, lb, accb);
        }
    }
    // the warps of the CTA, through shared memory, merged by warp 0 in order
    if (grp == 0) {
#pragma unroll
        for (int g = 0; g < GT; ++g) {
            if (sub == 0) {
                sm_m[warp][g] = m[g];
                sm_l[warp][g] = l[g];
            }
#pragma unroll
            for (int i = 0; i < 8; ++i) sm_acc[warp][g][sub * 8 + i] = acc[g][i];
        }
    }
    __syncthreads();
    if (warp != 0 || grp != 0) return;
#pragma unroll
    for (int w = 1; w < kDecodeWarps; ++w) {
        float mb[GT], lb[GT], accb[GT][8];
#pragma unroll
        for (int g = 0; g < GT; ++g) {
            mb[g] = sm_m[w][g];
            lb[g] = sm_l[w][g];
#pragma unroll
            for (int i = 0; i < 8; ++i) accb[g][i] = sm_acc[w][g][sub * 8 + i];
        }
        merge_streams<GT>(m, l, acc, mb, lb, accb);
    }
    if (!active) return;
#pragma unroll
    for (int g = 0; g < GT; ++g) {
        if (g >= gcount) continue;
        int hq = hk * G + g0 + g;
        if (n_splits == 1) {
            float inv = l[g] > 0.f ? 1.0f / l[g] : 0.f;
            bf16* o = out + ((size_t)n * nq + hq) * d + sub * 8;
            float4 a = make_float4(acc[g][0] * inv, acc[g][1] * inv, acc[g][2] * inv, acc[g][3] * inv);
            float4 b = make_float4(acc[g][4] * inv, acc[g][5] * inv, acc[g][6] * inv, acc[g][7] * inv);
            store4(o, a);
            store4(o + 4, b);
        } else {
            float* rec = partial + (((size_t)n * nq + hq) * n_splits + split) * (size_t)(d + 2);
            if (sub == 0) {
                rec[0] = m[g];
                rec[1] = l[g];
            }
#pragma unroll
            for (int i = 0; i < 8; ++i) rec[2 + sub * 8 + i] = acc[g][i];
        }
    }
}

template <int LPK, int GT>
static int launch_decode_final(dim3 grid, size_t smem, bool pdl, cudaStream_t stream, const bf16* q,
                               int q_stride, const bf16* k, const bf16* v, const int* pos,
                               const int* seq, const int* table, int cols, bf16* out, float* partial,
                               int nq, int nkv, int d, int page_size, int window, float scale,
                               int n_splits, int head_tiles, int stages, int* status) {
    auto kernel = attn_decode_kernel<LPK, GT>;
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             (int)smem);
        if (e != cudaSuccess) return (int)e;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(kDecodeWarps * 32);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 1 : 0;
    cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, q, q_stride, k, v, pos, seq, table, cols, out,
                                       partial, nq, nkv, d, page_size, window, scale, n_splits,
                                       head_tiles, stages, status);
    return e == cudaSuccess ? NNIS_OK : (int)e;
}

template <int LPK>
static int launch_decode_gt(int gt, dim3 grid, size_t smem, bool pdl, cudaStream_t stream,
                            const bf16* q, int q_stride, const bf16* k, const bf16* v, const int* pos,
                            const int* seq, const int* table, int cols, bf16* out, float* partial,
                            int nq, int nkv, int d, int page_size, int window, float scale,
                            int n_splits, int head_tiles, int stages, int* status) {
#define NNIS_DECODE_CASE(GT) \
    return launch_decode_final<LPK, GT>(grid, smem, pdl, stream, q, q_stride, k, v, pos, seq, table, \
                                        cols, out, partial, nq, nkv, d, page_size, window, scale, \
                                        n_splits, head_tiles, stages, status)
    switch (gt) {
        case 1: NNIS_DECODE_CASE(1);
        case 2: NNIS_DECODE_CASE(2);
        case 3: NNIS_DECODE_CASE(3);
        default: NNIS_DECODE_CASE(4);
    }
#undef NNIS_DECODE_CASE
}

}  // namespace nnis

// defined in attention_generic.cu
extern "C" int nnis_attention_merge_bf16(const float* partial, void* out, long long n_rows, int d,
                                         int n_splits, cudaStream_t stream);

// Scratch: `partial` needs n_tokens * nq * n_splits * (d + 2) floats when
// n_splits > 1 and may be null otherwise.  With `merge == 0` the partial records
// are left for a later kernel to merge (the output projection's prologue).
NNIS_API int nnis_attention_decode(const void* q, int q_stride, const void* k_cache,
                                   const void* v_cache, const int* token_pos, const int* token_seq,
                                   const int* page_table, int table_cols, void* out, float* partial,
                                   int n_tokens, int nq, int nkv, int d, int page_size, int window,
                                   float scale, int n_splits, int merge, int* status, int pdl,
                                   cudaStream_t stream) {
    using namespace nnis;
    if (n_tokens <= 0 || nq <= 0 || nkv <= 0 || nq % nkv || page_size <= 0 || table_cols <= 0 ||
        n_splits <= 0 || window < 0)
        return NNIS_ERR_ARGUMENT;
    if (d <= 0 || d % 16 || d > 256) return NNIS_ERR_UNSUPPORTED;
    if (n_tokens > 65535 || n_splits > 65535) return NNIS_ERR_UNSUPPORTED;
    if (n_splits > 1 && !partial) return NNIS_ERR_ARGUMENT;
    if (((uintptr_t)q | (uintptr_t)k_cache | (uintptr_t)v_cache | (uintptr_t)out) % 16 ||
        (q_stride % 8))
        return NNIS_ERR_ALIGNMENT;
    int G = nq / nkv;
    int gt = G < 4 ? G : 4;
    int head_tiles = (G + gt - 1) / gt;
    dim3 grid(nkv * head_tiles, n_tokens, n_splits);
    size_t stage_bytes = 2 * (size_t)page_size * d * sizeof(bf16);
    if (stage_bytes % 32) return NNIS_ERR_UNSUPPORTED;
    int stages = (int)((96 * 1024) / stage_bytes);
    stages = stages < 2 ? 2 : (stages > 8 ? 8 : stages);
    size_t smem = stages * stage_bytes + stages * sizeof(uint64_t);
    if (smem > 200 * 1024) return NNIS_ERR_UNSUPPORTED;
    int rc;
    const bf16* qp = (const bf16*)q;
    const bf16* kp = (const bf16*)k_cache;
    const bf16* vp = (const bf16*)v_cache;
#define NNIS_DECODE_LPK(LPK) \
    rc = launch_decode_gt<LPK>(gt, grid, smem, pdl != 0, stream, qp, q_stride, kp, vp, token_pos, \
                               token_seq, page_table, table_cols, (bf16*)out, partial, nq, nkv, d, \
                               page_size, window, scale, n_splits, head_tiles, stages, status)
    if (d <= 16) NNIS_DECODE_LPK(2);
    else if (d <= 32) NNIS_DECODE_LPK(4);
    else if (d <= 64) NNIS_DECODE_LPK(8);
    else if (d <= 128) NNIS_DECODE_LPK(16);
    else NNIS_DECODE_LPK(32);
#undef NNIS_DECODE_LPK
    if (rc != NNIS_OK) return rc;
    if (n_splits > 1 && merge)
        return nnis_attention_merge_bf16(partial, out, (long long)n_tokens * nq, d, n_splits, stream);
    return NNIS_OK;
}
