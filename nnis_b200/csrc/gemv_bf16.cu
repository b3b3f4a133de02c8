// Entry point of the decode projections (see gemv_kernel.cuh for the kernel):
// picks the launch shape for a problem and hands it to the instantiation for its
// number of 16-row tiles of x (gemv_tiles1.cu .. gemv_tiles4.cu).
#include <stdlib.h>

#include "gemv_kernel.cuh"

namespace nnis {

int gemv_launch_tiles1(const GemvArgs&, int, int, const GemvPlan&, bool, cudaStream_t);
int gemv_launch_tiles2(const GemvArgs&, int, int, const GemvPlan&, bool, cudaStream_t);
int gemv_launch_tiles3(const GemvArgs&, int, int, const GemvPlan&, bool, cudaStream_t);
int gemv_launch_tiles4(const GemvArgs&, int, int, const GemvPlan&, bool, cudaStream_t);
// gemv_rowtile.cu: the kernel for more rows than one tile and few output features
int gemv_rowtile_units(int M, int N, int K, int epilogue, int pro, int sm_count);
int gemv_launch_rowtile(const GemvArgs&, int, int, int, bool, cudaStream_t);

// Shared memory of one CTA: x, the weight stages (eight rows of `kc` columns each),
// the barriers, and with split K the warps' partial sums.
static size_t gemv_smem(int mtiles, int warps, int stages, int K, int kc, bool splitk) {
    size_t sets = splitk ? 1 : (size_t)warps * stages;
    return ((size_t)mtiles * 16 * (K + 8) + sets * 8 * (kc + 8)) * sizeof(bf16) +
           (size_t)warps * stages * 8 + (splitk ? (size_t)warps * mtiles * 4 * 32 * sizeof(float) : 0);
}

static int env_int(const char* name, int fallback) {
    const char* v = getenv(name);
    return v && *v ? atoi(v) : fallback;
}

static bool gemv_plan(int M, int N, int K, int sm_count, GemvPlan* plan) {
    if (M <= 0 || M > 64 || K <= 0 || K % 16 || N <= 0 || N % 8) return false;
    int sms = sm_count > 0 ? sm_count : 148;
    int mtiles = (M + 15) / 16;
    int units = N / 8;
    const size_t budget = 200 * 1024;
    static const int chunk_min_k = env_int("NNIS_GEMV_CHUNK_MIN_K", 2048);
    static const int chunk_cols = env_int("NNIS_GEMV_CHUNK_COLS", 512);
    plan->kc = K;
    // Few units: one per CTA, its eight warps sharing K.
    {
        size_t smem = gemv_smem(mtiles, 8, 1, K, K, true);
        size_t per_sm = smem + 1024;
        int fit = (int)((220 * 1024) / per_sm);
        if (fit > 8) fit = 8;
        if (smem <= budget && fit >= 1 && units <= sms * fit) {
            plan->mtiles = mtiles; plan->warps = 8; plan->stages = 1; plan->grid = units;
            plan->splitk = true; plan->smem = smem;
            return true;
        }
    }
    for (int warps = 8; warps >= 4 && K < chunk_min_k; warps -= 4) {
        // Many units: as many CTAs as fit (units are dealt to CTAs first), each
        // warp streaming its own units through one or two stages.
        for (int stages = 2; stages >= 1; --stages) {
            size_t smem = gemv_smem(mtiles, warps, stages, K, K, false);
            if (smem > budget) continue;
            int cap = smem > 110 * 1024 ? sms : sms * 2;
            int grid = units < cap ? units : cap;
            bool many = units > grid * warps;  // some warp has several units
            if (stages == 2 && (!many || smem > 100 * 1024)) continue;
            plan->mtiles = mtiles; plan->warps = warps; plan->stages = stages; plan->grid = grid;
            plan->splitk = false; plan->smem = smem;
            return true;
        }
    }
    // Long rows: a stage holds a chunk of K, two stages per warp, so that the
    // copies of the next chunk run under the products of this one.
    for (int kc = chunk_cols; kc >= 128; kc >>= 1) {
        if (kc >= K) continue;
        size_t smem = gemv_smem(mtiles, 8, 2, K, kc, false);
        if (smem > budget) continue;
        int cap = smem > 110 * 1024 ? sms : sms * 2;
        plan->mtiles = mtiles; plan->warps = 8; plan->stages = 2; plan->grid = units < cap ? units : cap;
        plan->splitk = false; plan->smem = smem; plan->kc = kc;
        return true;
    }
    return false;
}

// In how many slices of K a product with the ADD_F32 epilogue runs (each slice
// a launch that adds its share into the output, in order): 1 when the kernel
// takes the whole K, 0 when no slicing helps.  Rows of x longer than shared
// memory are the reason: the kernel keeps all of x there.
static int gemv_slices(int M, int N, int K, int sm_count, GemvPlan* plan) {
    if (gemv_plan(M, N, K, sm_count, plan) && (plan->splitk || plan->kc == K)) return 1;
    // Few output rows and long rows of K: slices short enough for the launch shape
    // whose warps share K are faster than chunks that leave most warps without a unit.
    int first = plan->kc != K ? 1 : 0;
    for (int c = 2; c <= 16; ++c) {
        if (K % (16 * c)) continue;
        GemvPlan p;
        if (!gemv_plan(M, N, K / c, sm_count, &p)) continue;
        if (p.splitk) {
            *plan = p;
            return c;
        }
        if (!first) first = c;
    }
    if (first && gemv_plan(M, N, K / first, sm_count, plan)) return first;
    return 0;
}

// The kernel over tiles of rows: in how many slices of K it runs a product (0: it does
// not take it), and with how many units per CTA.  Only the adding epilogue may be cut:
// each slice a launch that adds its share into the output, in order.
static int rowtile_slices(int M, int N, int K, int epilogue, int pro, int sm_count, int* units) {
    *units = gemv_rowtile_units(M, N, K, epilogue, pro, sm_count);
    if (*units > 0) return 1;
    if (epilogue != EPI_ADD_F32 || pro != PRO_PLAIN) return 0;
    for (int c = 2; c <= 3; ++c) {  // (more launches than that cost more than the general kernel)
        if (K % (16 * c)) continue;
        *units = gemv_rowtile_units(M, N, K / c, epilogue, pro, sm_count);
        if (*units > 0) return c;
    }
    return 0;
}

}  // namespace nnis

// Whether nnis_gemv_bf16 takes a shape (1) or the caller must use the general
// kernels (0): at most 64 rows, K a multiple of 16, N a multiple of 8, and x plus
// the weight stages must fit shared memory.
NNIS_API int nnis_gemv_takes(int M, int N, int K, int sm_count) {
    nnis::GemvPlan p;
    return nnis::gemv_plan(M, N, K, sm_count, &p) ? 1 : 0;
}

// Slices of K for the ADD_F32 epilogue with a plain prologue: 0 not taken, 1 one
// launch, more: that many launches inside nnis_gemv_bf16.
NNIS_API int nnis_gemv_slices(int M, int N, int K, int sm_count) {
    nnis::GemvPlan p;
    int units;
    int rows = nnis::rowtile_slices(M, N, K, nnis::EPI_ADD_F32, nnis::PRO_PLAIN, sm_count, &units);
    return rows > 0 ? rows : nnis::gemv_slices(M, N, K, sm_count, &p);
}

// Which kernel nnis_gemv_bf16 runs for a product: 2 the one that cuts the rows into
// tiles (gemv_rowtile.cu: more than 16 rows, few output features), 1 the one whose
// CTAs hold all rows (at most 64), 0 neither.  `normed`: the prologue (0 x as it is, 1
// the norm, 2 x weighted and the rows' sums of squares in shares: the first kernel only).
NNIS_API int nnis_gemv_kind(int M, int N, int K, int epilogue, int normed, int sm_count) {
    using namespace nnis;
    int units;
    const int pro = normed == 2 ? PRO_SCALED : normed ? PRO_NORM : PRO_PLAIN;
    if (rowtile_slices(M, N, K, epilogue, pro, sm_count, &units) > 0) return 2;
    if (pro == PRO_SCALED) return 0;
    GemvPlan p;
    if (epilogue == EPI_ADD_F32 && !normed) return gemv_slices(M, N, K, sm_count, &p) >= 1 ? 1 : 0;
    return gemv_plan(M, N, K, sm_count, &p) ? 1 : 0;
}

// The same questions for the kernel whose CTAs hold all rows alone (what bit 2 of
// nnis_gemv_bf16's `pdl` selects).
NNIS_API int nnis_gemv_units_takes(int M, int N, int K, int epilogue, int normed, int sm_count) {
    nnis::GemvPlan p;
    if (epilogue == nnis::EPI_ADD_F32 && !normed) return nnis::gemv_slices(M, N, K, sm_count, &p) >= 1 ? 1 : 0;
    return nnis::gemv_plan(M, N, K, sm_count, &p) ? 1 : 0;
}

NNIS_API int nnis_gemv_units_slices(int M, int N, int K, int sm_count) {
    nnis::GemvPlan p;
    return nnis::gemv_slices(M, N, K, sm_count, &p);
}

// How many CTAs a launch with these sizes has: the ARGMAX scratch is
// [M, this many] values and indices.
NNIS_API int nnis_gemv_grid(int M, int N, int K, int sm_count) {
    nnis::GemvPlan p;
    return nnis::gemv_plan(M, N, K, sm_count, &p) ? p.grid : 0;
}

// Scratch: the ARGMAX epilogue uses `best_val`, `best_idx` ([M, nnis_gemv_grid()]
// each) and `ticket` (one zeroed counter, left zero).  `pdl`: bit 0 launches the kernel
// as a programmatic dependent of the one before it; bit 1 lets the kernel after it
// start together with this one (only for a successor that reads nothing of this step
// before its own wait); bit 2: not the kernel over tiles of rows, even where it applies
// (for comparisons).
// `emit_x`, `emit_w`, `emit_ss` (ADD_F32, optional): the output rows times the weights
// `emit_w` [N] in bfloat16 [M, N], and per row and eight columns the sum of the output's
// squares [M, N / 8], for a product that follows with `ss_parts` [M, K / 8]: x is then such
// an `emit_x`, and `eps` the norm's (the kernel over tiles of rows only).
NNIS_API int nnis_gemv_bf16(const void* x, const float* hidden, const int* rows, const float* norm_w,
                            float eps, const void* w, const float* bias, void* out, int M, int N,
                            int K, int epilogue, const int* token_pos, const int* token_seq,
                            const int* page_table, int table_cols, const float* cos_t,
                            const float* sin_t, void* k_cache, void* v_cache, int nq, int nkv, int d,
                            int page_size, float* logits, float* best_val, int* best_idx,
                            unsigned* ticket, int* next_tokens, int* next_pos, void* emit_x,
                            const float* emit_w, float* emit_ss, const float* ss_parts, int* status,
                            int sm_count, int pdl, cudaStream_t stream) {
    using namespace nnis;
    if (M <= 0 || N <= 0 || K <= 0 || !w || !out) return NNIS_ERR_ARGUMENT;
    GemvPlan plan;
    plan.kc = K;
    int pro = hidden ? PRO_NORM : ss_parts ? PRO_SCALED : PRO_PLAIN;
    if (hidden && ss_parts) return NNIS_ERR_ARGUMENT;
    if (emit_x && (epilogue != EPI_ADD_F32 || !emit_w || !emit_ss)) return NNIS_ERR_ARGUMENT;
    if (((uintptr_t)emit_x | (uintptr_t)emit_w) % 8) return NNIS_ERR_ALIGNMENT;
    // more rows than a tile and few output features: the kernel that cuts the rows
    int rowtile_units = 0;
    const int rowtile_cuts = (pdl & 4) ? 0 : rowtile_slices(M, N, K, epilogue, pro, sm_count, &rowtile_units);
    const bool may_slice = epilogue == EPI_ADD_F32 && pro == PRO_PLAIN;
    const int slices = rowtile_cuts > 0 ? rowtile_cuts
                       : may_slice      ? gemv_slices(M, N, K, sm_count, &plan)
                                        : (gemv_plan(M, N, K, sm_count, &plan) ? 1 : 0);
    if (slices == 0) return NNIS_ERR_UNSUPPORTED;
    if (pro != PRO_NORM && !x) return NNIS_ERR_ARGUMENT;
    if (pro == PRO_NORM && (!norm_w || !(eps > 0.f))) return NNIS_ERR_ARGUMENT;
    if (pro == PRO_SCALED && (rowtile_cuts != 1 || !(eps > 0.f))) return NNIS_ERR_UNSUPPORTED;
    if (((uintptr_t)w | (uintptr_t)x | (uintptr_t)hidden | (uintptr_t)norm_w) % 16 ||
        (uintptr_t)out % (epilogue == EPI_ARGMAX ? 4 : 16))  // the picks are single words
        return NNIS_ERR_ALIGNMENT;
    if (epilogue == EPI_QKV) {
        if (!token_pos || d <= 0 || d % 8 || N != (nq + 2 * nkv) * d) return NNIS_ERR_ARGUMENT;
        if (nkv > 0 && (!token_seq || !page_table || !k_cache || !v_cache || page_size <= 0))
            return NNIS_ERR_ARGUMENT;
    }
    if (epilogue == EPI_ARGMAX && (!best_val || !best_idx || !ticket)) return NNIS_ERR_ARGUMENT;
    if (epilogue == EPI_ARGMAX && next_tokens && !next_pos) return NNIS_ERR_ARGUMENT;
    GemvArgs a;
    a.x = (const bf16*)x; a.hidden = hidden; a.rows = rows; a.norm_w = norm_w; a.eps = eps;
    a.w = (const bf16*)w; a.bias = bias; a.out = out; a.M = M; a.N = N; a.K = K; a.status = status;
    a.token_pos = token_pos; a.token_seq = token_seq; a.page_table = page_table;
    a.table_cols = table_cols; a.cos_t = cos_t; a.sin_t = sin_t; a.k_cache = (bf16*)k_cache;
    a.v_cache = (bf16*)v_cache; a.nq = nq; a.nkv = nkv; a.d = d > 0 ? d : 8; a.page_size = page_size;
    a.logits = logits; a.best_val = best_val; a.best_idx = best_idx; a.ticket = ticket;
    a.next_tokens = next_tokens; a.next_pos = next_pos;
    a.emit_x = nullptr; a.emit_w = emit_w; a.emit_ss = emit_ss;
    a.ss_parts = ss_parts; a.ss_units = K / 8;
    a.ldx = K; a.ldw = K; a.kc = plan.kc; a.out_is_hot = 0;
    a.release_early = (pdl & 2) && slices == 1 ? 1 : 0;
    a.K = K / slices;
    static const char* const kNames[] = {"gemv store", "gemv store_f32", "gemv add_f32", "gemv gated",
                                         "gemv qkv", "gemv argmax"};
    static const char* const kRowNames[] = {"gemv rows store", "gemv rows store_f32", "gemv rows add_f32",
                                            "gemv rows gated", "gemv rows qkv"};
    for (int s = 0; s < slices; ++s) {
        int rc;
        if (s == slices - 1) a.emit_x = (bf16*)emit_x;  // the sums are whole after the last slice
        if (rowtile_cuts > 0) {
            a.trace = trace_slot(epilogue >= 0 && epilogue <= 4 ? kRowNames[epilogue] : "gemv rows");
            rc = gemv_launch_rowtile(a, epilogue, pro, rowtile_units, (pdl & 1) != 0, stream);
        } else {
        a.trace = trace_slot(epilogue >= 0 && epilogue <= 5 ? kNames[epilogue] : "gemv");
        switch (plan.mtiles) {
            case 1: rc = gemv_launch_tiles1(a, epilogue, pro, plan, (pdl & 1) != 0, stream); break;
            case 2: rc = gemv_launch_tiles2(a, epilogue, pro, plan, (pdl & 1) != 0, stream); break;
            case 3: rc = gemv_launch_tiles3(a, epilogue, pro, plan, (pdl & 1) != 0, stream); break;
            default: rc = gemv_launch_tiles4(a, epilogue, pro, plan, (pdl & 1) != 0, stream); break;
        }
        }
        if (rc != NNIS_OK) return rc;
        a.x += a.K;
        a.w += a.K;
        a.bias = nullptr;  // the first slice has added it
        a.out_is_hot = 1;
    }
    return NNIS_OK;
}
