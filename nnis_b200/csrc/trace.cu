// A timeline of the kernels of a step, for measurements: when a trace buffer is set,
// every launch of an instrumented kernel takes the next slot of eight 64-bit words
// and its CTAs record, from the GPU's nanosecond timer,
//   [0] when the first CTA began          [1] when the last CTA ended
//   [2] when the first CTA got past its wait for the kernel before it
//   [3] when the last one did
//   [4], [5] first and last CTA at a first mark inside the kernel (projections: x is in
//            shared memory; attention: all pages of the slice are done)
//   [6], [7] the same for a second mark (projections: products done; attention: the
//            ticket is taken).
// A slot belongs to a launch for good (a captured graph writes the same slots at
// every replay), so the host clears the buffer, replays once and reads it.  With no
// buffer set (the normal case) kernels get a null pointer and record nothing.
#include "common.cuh"

namespace {
unsigned long long* g_buf = nullptr;
int g_capacity = 0, g_next = 0;
const char* g_names[4096];
}  // namespace

namespace nnis {
unsigned long long* trace_slot(const char* name) {
    if (!g_buf || g_next >= g_capacity || g_next >= 4096) return nullptr;
    g_names[g_next] = name;
    return g_buf + 8 * (size_t)(g_next++);
}
}  // namespace nnis

// `buffer`: device memory of 8 * capacity 64-bit words, or null to stop tracing.
NNIS_API void nnis_trace_set(void* buffer, int capacity) {
    g_buf = reinterpret_cast<unsigned long long*>(buffer);
    g_capacity = buffer ? capacity : 0;
    g_next = 0;
}

NNIS_API int nnis_trace_count() { return g_next; }

NNIS_API const char* nnis_trace_name(int slot) {
    return slot >= 0 && slot < g_next ? g_names[slot] : "";
}
