// Pieces shared by the tile SpMM kernels (tile_spmm.cu: per-warp cp.async rings, tcgen05
// variant; tile_gather4.cu: TMA gather ring): kernel arguments, unit-range search, MMA and
// mbarrier wrappers.
#pragma once

#include "tile_plan.cuh"

namespace ra {

struct TileArgs {
    const int* block_offsets;
    const int* atox;
    const uint16_t* vals;
    const unsigned long long* val_masks;   // zero-compressed plans (vals is null)
    const int* val_base;
    const uint16_t* vals_zc;
    const int* win_rows;
    const int* seg_window;
    const int* seg_bbegin;
    const int* seg_bend;
    const int* seg_scratch;
    int num_units;
    int M;
    int K;                     // rows of the B operand
    int N;
    int ldb;                   // row stride of the B operand in elements (N, or N rounded up to 16
                               // when the library made a padded fp16 copy)
    long long total_blocks;
    int max_unit_blocks;       // blocks of the longest unit (window, or 64 for segments)
    float* C;
    float* scratch;
    long long scratch_floats;     // capacity of scratch
};

__device__ __forceinline__ void cp_async_16(void* smem_dst, const void* gsrc) {
    const unsigned s = (unsigned)__cvta_generic_to_shared(smem_dst);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" :: "r"(s), "l"(gsrc) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int kPending>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" :: "n"(kPending) : "memory"); }

__device__ __forceinline__ void mma_f16_m16n8k8(float (&d)[4], unsigned a0, unsigned a1, unsigned b0) {
    asm volatile("mma.sync.aligned.m16n8k8.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5}, {%6}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3]) : "r"(a0), "r"(a1), "r"(b0));
}
__device__ __forceinline__ void mma_tf32_m16n8k8(float (&d)[4], unsigned a0, unsigned a1, unsigned a2,
                                                 unsigned a3, unsigned b0, unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ unsigned to_tf32_rna(float x) {
    unsigned r = __float_as_uint(x);
    asm("cvt.rna.tf32.f32 %0, %0;" : "+r"(r));
    return r;
}

// Zero-compressed value of (vector k, window row r) of a block: bit k*8+r of the mask says
// whether it is stored; stored values are packed in bit order from `base` on
// (same format as zc_val_bits, tc/ra_tc_direct.cu:402-414).
__device__ __forceinline__ unsigned zc_value_bits(unsigned long long mask, int base,
                                                  const uint16_t* __restrict__ vals_zc, int k, int r) {
    const int bit = k * 8 + r;
    if (!((mask >> bit) & 1ull)) return 0u;
    const unsigned long long below = mask & ((1ull << bit) - 1ull);
    return (unsigned)__ldg(vals_zc + base + __popcll(below));
}

// first block of unit u (u == num_units gives the total)
template <int kMode>
__device__ __forceinline__ long long unit_begin(const TileArgs& a, int u) {
    if (u >= a.num_units) return a.total_blocks;
    return (kMode == 2) ? (long long)__ldg(a.seg_bbegin + u) : (long long)__ldg(a.block_offsets + u);
}
template <int kMode>
__device__ __forceinline__ int unit_lower_bound(const TileArgs& a, long long target) {
    int lo = 0, hi = a.num_units;          // smallest u with unit_begin(u) + u >= target
    while (lo < hi) {
        const int mid = (lo + hi) >> 1;
        if (unit_begin<kMode>(a, mid) + mid < target) lo = mid + 1; else hi = mid;
    }
    return lo;
}

__device__ __forceinline__ void mma_f16_m16n8k16(float (&d)[4], unsigned a0, unsigned a1, unsigned a2,
                                                 unsigned a3, unsigned b0, unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}


constexpr int kSpinLimit = 1 << 22;
enum { kStatusFullTimeout = 1, kStatusEmptyTimeout = 2 };

__device__ __forceinline__ void mbar_init(unsigned addr, int count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" :: "r"(addr), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(unsigned addr, unsigned bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" :: "r"(addr), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(unsigned addr) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" :: "r"(addr) : "memory");
}
__device__ __forceinline__ bool mbar_wait(unsigned addr, unsigned parity, int limit = kSpinLimit) {
    for (int i = 0; i < limit; ++i) {
        unsigned ok;
        asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                     : "=r"(ok) : "r"(addr), "r"(parity) : "memory");
        if (ok) return true;
    }
    return false;
}
// Whole-warp form: the 32 lanes poll together and agree on the outcome, so the code after the
// wait (warp-synchronous shared-memory reads) never runs with a part of the warp.
__device__ __forceinline__ bool mbar_wait_warp(unsigned addr, unsigned parity, int limit) {
    for (int i = 0; i < limit; ++i) {
        unsigned ok;
        asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                     : "=r"(ok) : "r"(addr), "r"(parity) : "memory");
        if (__all_sync(0xffffffffu, ok != 0u)) return true;
    }
    return false;
}
// As mbar_wait_warp with a suspend-time hint (ns) on every poll: the hardware may park the
// thread until the barrier completes or the hint expires. hint_ns == 0 polls without a hint.
__device__ __forceinline__ bool mbar_wait_warp_hint(unsigned addr, unsigned parity, int limit, unsigned hint_ns) {
    if (hint_ns == 0u) return mbar_wait_warp(addr, parity, limit);
    for (int i = 0; i < limit; ++i) {
        unsigned ok;
        asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                     : "=r"(ok) : "r"(addr), "r"(parity), "r"(hint_ns) : "memory");
        if (__all_sync(0xffffffffu, ok != 0u)) return true;
    }
    return false;
}
__device__ __forceinline__ void bulk_copy_g2s(unsigned dst, const void* src, unsigned bytes, unsigned mbar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 :: "r"(dst), "l"(src), "r"(bytes), "r"(mbar) : "memory");
}

// TMA gather ring (tile_gather4.cu). RA_ERR_UNSUPPORTED = shape not covered, use another kernel.
template <bool kTF32, int kMode>
int launch_tile_gather4(const TileArgs& a, const void* B, long long K, cudaStream_t st, int* status);
// floats of scratch that lets the ring share windows between groups (0: not applicable)
long long tile_gather4_split_scratch_floats(bool tf32, int mode, const TileArgs& a);

}  // namespace ra
