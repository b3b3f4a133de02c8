// Decode attention for callers that cannot allocate: the split-KV scratch of
// nnis_attention_decode_mma lives in a fixed device array of this file.  See
// no_alloc.h for who needs this, the limits and the rules.
#include <mutex>

#include "common.cuh"
#include "no_alloc.h"

// defined in attention_decode_mma.cu
extern "C" int nnis_attention_decode_mma(const void* q, int q_stride, const void* k_cache,
                                         const void* v_cache, const int* token_pos,
                                         const int* token_seq, const int* page_table, int table_cols,
                                         void* out, float* partial, unsigned* tickets, int n_tokens,
                                         int nq, int nkv, int d, int page_size, int window,
                                         float scale, int n_splits, int pdl, cudaStream_t stream);

// Partial records first, tickets after them.  In host code this name is only a
// handle for cudaGetSymbolAddress; the device address is looked up per device.
static __device__ __align__(256) unsigned char nnis_noalloc_scratch[NNIS_NOALLOC_SCRATCH_BYTES];

namespace {
constexpr int kMaxDevices = 64;
void* g_scratch[kMaxDevices] = {};
std::mutex g_mutex;

// The array's address on the current device; looked up on the first call there.
int scratch_address(void** ptr) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int)e;
    if (dev < 0 || dev >= kMaxDevices) return NNIS_ERR_UNSUPPORTED;
    std::lock_guard<std::mutex> lock(g_mutex);
    if (!g_scratch[dev]) {
        void* p = nullptr;
        e = cudaGetSymbolAddress(&p, nnis_noalloc_scratch);
        if (e != cudaSuccess) return (int)e;
        if (!p) return NNIS_ERR_ARGUMENT;
        g_scratch[dev] = p;
    }
    *ptr = g_scratch[dev];
    return NNIS_OK;
}
}  // namespace

NNIS_API int nnis_attention_decode_noalloc(const void* q, int q_stride, const void* k_cache,
                                           const void* v_cache, const int* token_pos,
                                           const int* token_seq, const int* page_table,
                                           int table_cols, void* out, int n_tokens, int heads,
                                           int kv_heads, int head_dim, int page_size, int window,
                                           float scale, int n_splits, cudaStream_t stream) {
    // Everything the kernel's own entry point would refuse is refused here first, so
    // that a refused call puts nothing on the stream (not even the clearing below).
    if (n_tokens <= 0 || heads <= 0 || kv_heads <= 0 || heads % kv_heads || n_splits <= 0 ||
        head_dim <= 0 || table_cols <= 0 || window < 0)
        return NNIS_ERR_ARGUMENT;
    if ((head_dim != 64 && head_dim != 128) || page_size != 64 || n_tokens > 65535 || n_splits > 64)
        return NNIS_ERR_UNSUPPORTED;
    if (((uintptr_t)q | (uintptr_t)k_cache | (uintptr_t)v_cache | (uintptr_t)out) % 16 ||
        (q_stride % 8))
        return NNIS_ERR_ALIGNMENT;
    unsigned long long floats =
        (unsigned long long)n_tokens * heads * n_splits * (unsigned long long)(head_dim + 2);
    unsigned long long tickets =
        (unsigned long long)n_tokens * kv_heads * ((heads / kv_heads + 15) / 16);
    if (floats > NNIS_NOALLOC_PARTIAL_FLOATS || tickets > NNIS_NOALLOC_TICKETS)
        return NNIS_ERR_NOALLOC_TOO_LARGE;
    void* base = nullptr;
    int rc = scratch_address(&base);
    if (rc != NNIS_OK) return rc;
    float* partial = reinterpret_cast<float*>(base);
    unsigned* ticket_words = reinterpret_cast<unsigned*>(reinterpret_cast<unsigned char*>(base) +
                                                        (size_t)NNIS_NOALLOC_PARTIAL_FLOATS * 4u);
    // the tickets must start at zero; the last call may have left them otherwise
    // only if it was cut short, but clearing costs one small memset on the stream
    // (a single slice takes no ticket)
    if (n_splits > 1) {
        cudaError_t e = cudaMemsetAsync(ticket_words, 0, (size_t)tickets * sizeof(unsigned), stream);
        if (e != cudaSuccess) return (int)e;
    }
    return nnis_attention_decode_mma(q, q_stride, k_cache, v_cache, token_pos, token_seq, page_table,
                                     table_cols, out, partial, ticket_words, n_tokens, heads, kv_heads,
                                     head_dim, page_size, window, scale, n_splits, /*pdl=*/0, stream);
}
