// Pieces shared by the kernels that run on the fifth-generation tensor cores:
// TMA tile loads, tensor-memory allocation, tcgen05.mma / commit / ld, the shared
// memory and instruction descriptors, and tensor-map encoding on the host.
#pragma once

#include <cuda.h>

#include <mutex>

#include "async_copy.cuh"
#include "common.cuh"

namespace nnis {

// Asks for a tensor map ahead of its first use: the first TMA instruction that
// names a map otherwise waits some 1,500 cycles for the 128 bytes of the map itself.
__device__ __forceinline__ void prefetch_tensormap(const CUtensorMap* map) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(map) : "memory");
}

__device__ __forceinline__ void tma_load_2d(void* dst_smem, const CUtensorMap* map, int c0, int c1,
                                            uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(smem_addr(dst_smem)), "l"(map), "r"(c0), "r"(c1), "r"(smem_addr(bar))
        : "memory");
}

// shared -> global tile store, and the same as an addition into the destination
// (float32); both belong to the thread's current bulk group
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* map, int c0, int c1, const void* src_smem) {
    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%1, %2}], [%3];"
                 ::"l"(map), "r"(c0), "r"(c1), "r"(smem_addr(src_smem))
                 : "memory");
}
__device__ __forceinline__ void tma_add_2d(const CUtensorMap* map, int c0, int c1, const void* src_smem) {
    asm volatile("cp.reduce.async.bulk.tensor.2d.global.shared::cta.add.tile.bulk_group [%0, {%1, %2}], [%3];"
                 ::"l"(map), "r"(c0), "r"(c1), "r"(smem_addr(src_smem))
                 : "memory");
}
// closes the bulk group and waits until its stores have read their shared memory
__device__ __forceinline__ void tma_store_commit_wait() {
    asm volatile("cp.async.bulk.commit_group;" ::: "memory");
    asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
}

__device__ __forceinline__ void tmem_alloc(uint32_t* dst_smem, uint32_t columns) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                     smem_addr(dst_smem)),
                 "r"(columns)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t addr, uint32_t columns) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(addr), "r"(columns)
                 : "memory");
}
__device__ __forceinline__ void tc_fence_before() {
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
// The mbarrier gets one arrival when every tcgen05.mma issued so far by this
// thread has completed.
__device__ __forceinline__ void tc_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                     smem_addr(bar))
                 : "memory");
}
__device__ __forceinline__ void tc_mma(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                       uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// 32 columns of this thread's lane; `tmem_load_wait` before the values are used
__device__ __forceinline__ void tmem_load32_issue(uint32_t taddr, uint32_t (&v)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]),
          "=r"(v[7]), "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]),
          "=r"(v[14]), "=r"(v[15]), "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]),
          "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]),
          "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_load_wait() {
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_load32(uint32_t taddr, uint32_t (&v)[32]) {
    tmem_load32_issue(taddr, v);
    tmem_load_wait();
}

// Shared memory matrix descriptor of a K-major tile whose rows are 128 bytes
// (64 bfloat16) and 128-byte swizzled: 8-row groups 1024 bytes apart.
__device__ __forceinline__ uint64_t smem_desc_k128(uint32_t smem_byte_addr) {
    uint64_t desc = 0;
    desc |= (uint64_t)((smem_byte_addr >> 4) & 0x3FFF);   // start address, 16-byte units
    desc |= (uint64_t)1 << 16;                            // leading byte offset (unused with swizzle)
    desc |= (uint64_t)(1024 >> 4) << 32;                  // stride byte offset between 8-row groups
    desc |= (uint64_t)1 << 46;                            // descriptor version of sm_100
    desc |= (uint64_t)2 << 61;                            // SWIZZLE_128B
    return desc;
}

// The same tile `bytes` further on in shared memory (a multiple of 16 that does
// not carry out of the 14 address bits).  The one thread that issues the products
// runs alone, every dependent instruction at full latency: building a descriptor
// from an address costs it over a hundred cycles per product, this one add does
// not, so descriptors are built once before a loop and advanced inside it.
__device__ __forceinline__ uint64_t desc_advance(uint64_t desc, uint32_t bytes) {
    return desc + (uint64_t)(bytes >> 4);
}

// kind::f16 instruction descriptor: bfloat16 x bfloat16 -> float32, both K-major.
__host__ __device__ constexpr uint32_t instr_desc(int m, int n) {
    return (1u << 4)                    // accumulator float32
         | (1u << 7)                    // A bfloat16
         | (1u << 10)                   // B bfloat16
         | ((uint32_t)(n >> 3) << 17)   // N / 8
         | ((uint32_t)(m >> 4) << 24);  // M / 16
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static inline EncodeTiledFn encode_tiled() {
    static EncodeTiledFn fn = nullptr;
    static bool tried = false;
    if (!tried) {
        tried = true;
        void* p = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) ==
                cudaSuccess && qres == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    }
    return fn;
}

// [rows, K] row-major bfloat16 or float32 (`elem_bytes` 2 or 4; rows `row_stride`
// elements apart; 0: packed), boxes of box_rows x 128 bytes, 128-byte swizzle.  Encoding a map costs the host a
// microsecond or two and a step encodes hundreds (weights, caches and workspace
// buffers at the same addresses every time), so the last maps are kept by key.
struct MapKey {
    const void* ptr;
    long long rows, row_stride;
    int K, box_rows, elem_bytes;
    bool operator==(const MapKey& o) const {
        return ptr == o.ptr && rows == o.rows && row_stride == o.row_stride && K == o.K &&
               box_rows == o.box_rows && elem_bytes == o.elem_bytes;
    }
};

static inline bool make_map(CUtensorMap* map, const void* ptr, long long rows, int K, int box_rows,
                            long long row_stride = 0, int elem_bytes = 2) {
    constexpr int kSlots = 512;
    struct Slot { MapKey key; CUtensorMap map; bool used; };
    static Slot slots[kSlots];
    static std::mutex lock;
    const MapKey key{ptr, rows, row_stride, K, box_rows, elem_bytes};
    size_t h = (size_t)((uintptr_t)ptr >> 4) * 0x9E3779B97F4A7C15ull;
    h ^= (size_t)rows * 0xC2B2AE3D27D4EB4Full + (size_t)K * 0x165667B19E3779F9ull + (size_t)box_rows * 31u +
         (size_t)row_stride * 0x27D4EB2F165667C5ull + (size_t)elem_bytes;
    Slot& slot = slots[(h >> 20) % kSlots];
    std::lock_guard<std::mutex> guard(lock);
    if (slot.used && slot.key == key) {
        *map = slot.map;
        return true;
    }
    EncodeTiledFn fn = encode_tiled();
    if (!fn) return false;
    cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)(row_stride > 0 ? row_stride : K) * (cuuint64_t)elem_bytes};
    cuuint32_t box[2] = {128u / (cuuint32_t)elem_bytes, (cuuint32_t)box_rows};  // one 128-byte swizzle row
    cuuint32_t elem[2] = {1, 1};
    if (fn(map, elem_bytes == 4 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, elem,
           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
        return false;
    slot.key = key;
    slot.map = *map;
    slot.used = true;
    return true;
}

}  // namespace nnis
