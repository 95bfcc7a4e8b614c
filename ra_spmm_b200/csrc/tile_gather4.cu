// Tile SpMM with the gathered B rows fetched by the Tensor Memory Accelerator.
//
// Same work and numerics as tile_spmm_kernel (tile_spmm.cu; replaces the kernels of
// tc/ra_tc_direct.cu:109-395, tc/ra_community_tc.cu:105-300 and
// tc/ra_segment_hybrid.cu:75-330): per 8-vector block the 8 gathered rows of B meet the packed
// sparse 8x8 block in one tensor-core MMA (FP16: two blocks per m16n8k16), fp32 accumulation
// in block order. What differs is who moves the bytes. The cp.async ring spends most of its
// issue slots on the gather itself (one 16-byte copy per lane and 8 rows, index shuffles,
// address arithmetic); here the rows of a block arrive through
//     cp.async.bulk.tensor.2d ... tile::gather4
// - four indexed rows of B per instruction, issued by a single lane, completion counted in
// bytes on an mbarrier - so a warp issues a handful of instructions per block and the loads
// cost no issue slots while they are in flight.
//
// Layout. B is described by one 2-D tensor map (inner dimension = a row of B, outer = the K
// rows) with a box of 128 bytes x 1 row and the 128-byte swizzle. A warp owns `S` column
// slices of 128 bytes (32 fp32 or 64 fp16 features) and a private ring of `D` stages; a stage
// holds, per slice, one 1 KB swizzle atom = the 8 gathered rows of a block (two gather4
// copies of 4 rows), plus the block's 128-byte packed values (one bulk copy; loading them
// into registers ahead of use instead was measured 15-30 % slower). The tensor-core
// k index j reads shared-memory row 2j (j < 4) or 2(j-4)+1 (j >= 4): with that interleave and
// the hardware swizzle (16-byte chunk index XOR row index) the 128-bit fragment loads of the
// TF32 path and the ldmatrix loads of the FP16 path are free of bank conflicts.
//
// Every wait is bounded: a warp whose stage never fills records the status word, collects
// (under the same bound) the copies it still has in flight, and returns.
//
// Work division. The units (windows, or segments of SEGMENT_HYBRID) lie on one axis where unit u
// with nb blocks occupies nb + 1 positions (its blocks, then its flush). Segments are at most 64
// blocks, so a group takes a run of whole segments. Windows can be thousands of blocks long (one
// window of 8 hub rows, or simply 490-block windows when a rank's share is two windows per
// group), so for the window families the axis is cut into equal pieces wherever the cut falls:
// a group may start and end inside a window. The part of a window that a group does not own
// completely goes to a partial tile in scratch (two slots per group: the window it entered
// through, the window it left through), and g4_chain_merge_kernel adds the partial tiles of a
// window in block order - always the same order, so the result is reproducible - and writes its rows.
#include "tile_common.cuh"

#include <cuda.h>

#include <algorithm>
#include <cstdlib>

namespace ra {

constexpr int kG4AtomBytes = 1024;      // 8 rows x 128 bytes
constexpr int kG4ValBytes  = 128;     // packed values of a block in the plan

// L2 eviction policies. The plan (packed values + gather indices, 160 bytes per block) is a
// stream that is read once per SpMM and is several times larger than the L2; the rows of B
// are what the L2 can serve again. The stream is therefore loaded evict-first and the rows of B
// evict-last, and C is written with streaming stores.
__device__ __forceinline__ unsigned long long l2_policy_evict_first() {
    unsigned long long p;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
    return p;
}
__device__ __forceinline__ unsigned long long l2_policy_normal() {
    unsigned long long p;
    asm volatile("createpolicy.fractional.L2::evict_normal.b64 %0, 1.0;" : "=l"(p));
    return p;
}
__device__ __forceinline__ unsigned long long l2_policy_evict_last() {
    unsigned long long p;
    asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(p));
    return p;
}

__device__ __forceinline__ void tma_gather4(unsigned dst, const CUtensorMap* map, int x,
                                            int r0, int r1, int r2, int r3, unsigned mbar,
                                            unsigned long long policy) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile::gather4.mbarrier::complete_tx::bytes.L2::cache_hint "
                 "[%0], [%1, {%2, %3, %4, %5, %6}], [%7], %8;"
                 :: "r"(dst), "l"(map), "r"(x), "r"(r0), "r"(r1), "r"(r2), "r"(r3), "r"(mbar), "l"(policy) : "memory");
}
__device__ __forceinline__ void bulk_copy_g2s_hint(unsigned dst, const void* src, unsigned bytes, unsigned mbar,
                                                   unsigned long long policy) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;"
                 :: "r"(dst), "l"(src), "r"(bytes), "r"(mbar), "l"(policy) : "memory");
}
__device__ __forceinline__ int4 ld_stream_first_int4(const int4* p) {      // read-once data: evict first
    return __ldcs(p);
}

// shared-memory row of tensor-core k index j (see the header comment)
__device__ __forceinline__ int g4_row_of_k(int j) { return (j < 4) ? 2 * j : 2 * (j - 4) + 1; }

// Cut `w` of the work axis -> (unit U, absolute block Bk): everything before block Bk of unit U
// lies before the cut. A cut that falls on a unit's flush position moves to the start of the next
// unit, so Bk < unit_begin(U + 1) whenever Bk > unit_begin(U).
template <int kMode>
__device__ __forceinline__ void g4_cut(const TileArgs& a, long long w, int& U, long long& Bk) {
    const long long total_w = a.total_blocks + a.num_units;
    if (w >= total_w) { U = a.num_units; Bk = a.total_blocks; return; }
    int u = unit_lower_bound<kMode>(a, w);                       // smallest u with begin(u) + u >= w
    long long ub = unit_begin<kMode>(a, u);
    if (u < a.num_units && ub + u == w) { U = u; Bk = ub; return; }
    --u;                                                         // the cut is inside unit u
    const long long ub0 = unit_begin<kMode>(a, u);
    const long long off = w - (ub0 + u);                         // 1 .. nb(u)
    if (ub0 + off >= ub) { U = u + 1; Bk = ub; } else { U = u; Bk = ub0 + off; }
}

// kMode: 0 natural windows, 1 window-row table (COMMUNITY_TC), 2 segments (SEGMENT_HYBRID).
// split (modes 0 and 1): groups own equal pieces of the work axis and may share a window.
// S: 128-byte slices per warp. D: ring stages per warp.
template <bool kTF32, int kMode, int S, int D>
__global__ void __launch_bounds__(256)
tile_spmm_gather4_kernel(const __grid_constant__ CUtensorMap bmap, TileArgs a, int slices_total,
                         int warps_per_group, int groups_total, int* __restrict__ status, unsigned wait_hint_ns, int l2_policies,
                         int split)
{
    constexpr int kMT    = kTF32 ? 2 : 4;           // 16-feature MMA tiles per slice
    constexpr int kElem  = kTF32 ? 4 : 2;
    constexpr int kSlcF  = 128 / kElem;             // features per slice
    static_assert(D >= 2 && (D & (D - 1)) == 0, "ring depth is a power of two");
    extern __shared__ unsigned char smem_raw[];

    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    const int warps_cta = blockDim.x >> 5;
    const int groups_per_cta = warps_cta / warps_per_group;
    const int grp = warp / warps_per_group;
    const int part = warp - grp * warps_per_group;
    const int gid = blockIdx.x * groups_per_cta + grp;
    const bool has_work = grp < groups_per_cta && gid < groups_total;

    // ---- shared memory: [atoms of every warp][values of every warp][barriers of every warp]
    unsigned char* base = reinterpret_cast<unsigned char*>(
        (reinterpret_cast<uintptr_t>(smem_raw) + (kG4AtomBytes - 1)) & ~(uintptr_t)(kG4AtomBytes - 1));
    unsigned char* atoms = base + (size_t)warp * D * S * kG4AtomBytes;
    unsigned char* vals_sm = base + (size_t)warps_cta * D * S * kG4AtomBytes + (size_t)warp * D * kG4ValBytes;
    unsigned char* bars_sm = base + (size_t)warps_cta * D * (S * kG4AtomBytes + kG4ValBytes) + (size_t)warp * D * 8;
    const unsigned atoms_s = (unsigned)__cvta_generic_to_shared(atoms);
    const unsigned vals_s = (unsigned)__cvta_generic_to_shared(vals_sm);
    const unsigned bars_s = (unsigned)__cvta_generic_to_shared(bars_sm);
    if (lane == 0) {
        for (int s = 0; s < D; ++s) mbar_init(bars_s + 8 * s, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    __syncwarp();
    if (!has_work) return;

    // ---- this group's piece of the work axis (blocks + one flush position per unit) ----
    const long long total_w = a.total_blocks + a.num_units;
    int u_lo, u_hi;                                              // units [u_lo, u_hi) are touched
    long long B0, B1;                                            // absolute block range
    bool head_partial = false, tail_partial = false;            // first / last touched unit shared with a neighbour
    if (kMode != 2 && split) {
        int us, ue; long long bs, be;
        g4_cut<kMode>(a, total_w * gid / groups_total, us, bs);
        g4_cut<kMode>(a, total_w * (gid + 1) / groups_total, ue, be);
        tail_partial = ue < a.num_units && be > unit_begin<kMode>(a, ue);
        head_partial = us < a.num_units && bs > unit_begin<kMode>(a, us);
        u_lo = us; u_hi = tail_partial ? ue + 1 : ue;
        B0 = bs; B1 = be;
        if (part == 0 && lane == 0) {
            // for the merge: the window this group entered through and the one it leaves through (-1: none)
            int2* shared_windows = reinterpret_cast<int2*>(a.scratch + (size_t)2 * groups_total * kWindowRows * a.N);
            shared_windows[gid] = make_int2(head_partial ? us : -1, tail_partial ? ue : -1);
        }
    } else {
        u_lo = unit_lower_bound<kMode>(a, total_w * gid / groups_total);
        u_hi = unit_lower_bound<kMode>(a, total_w * (gid + 1) / groups_total);
        B0 = unit_begin<kMode>(a, u_lo); B1 = unit_begin<kMode>(a, u_hi);
    }
    if (u_lo >= u_hi) return;
    const int nb = (int)(B1 - B0);                               // blocks of this piece

    const int N = a.N;
    const int slice0 = part * S;                                 // first slice of this warp
    const int s_valid = min(S, slices_total - slice0);           // slices this warp really has
    if (s_valid <= 0) return;
    const int f0 = slice0 * kSlcF;                               // first feature of this warp
    const unsigned char* vals_base = reinterpret_cast<const unsigned char*>(a.vals) + (size_t)B0 * kG4ValBytes;
    const int4* atox4 = reinterpret_cast<const int4*>(a.atox + B0 * kVecPerBlock);
    const unsigned stage_tx = (unsigned)(s_valid * kG4AtomBytes + kG4ValBytes);

    // ---- producer side ----
    // Gather indices are read 32 blocks at a time (lane l holds the 8 columns of block
    // ibase + l, one coalesced 1 KB load per batch, the next batch already in flight), and the
    // lane that holds a block's columns issues that block's copies itself: no index shuffles,
    // and no load latency between two consecutive blocks.
    int4 ca = make_int4(0, 0, 0, 0), cb = ca, na = ca, nb4 = ca;
    int ibase = 0;
    auto load_batch = [&](int first, int4& x, int4& y) {
        const int blk = first + lane;
        if (blk < nb) { x = ld_stream_first_int4(atox4 + 2 * blk); y = ld_stream_first_int4(atox4 + 2 * blk + 1); }
    };
    load_batch(0, ca, cb);
    load_batch(32, na, nb4);
    const unsigned long long pol_stream = l2_policies ? l2_policy_evict_first() : l2_policy_normal();
    const unsigned long long pol_rows = l2_policies ? l2_policy_evict_last() : l2_policy_normal();

    auto fetch = [&](int rf) {                                   // rf: block index relative to B0
        if (rf >= ibase + 32) { ca = na; cb = nb4; ibase += 32; load_batch(ibase + 32, na, nb4); }
        if (lane == (rf & 31)) {
            const int st = rf & (D - 1);
            const unsigned bar = bars_s + 8 * st;
            mbar_expect_tx(bar, stage_tx);
            const unsigned dst = atoms_s + (unsigned)(st * S * kG4AtomBytes);
#pragma unroll
            for (int sl = 0; sl < S; ++sl) {
                if (sl < s_valid) {
                    // rows 0-3 of the atom = vectors 0,4,1,5; rows 4-7 = vectors 2,6,3,7
                    const int x = (slice0 + sl) * kSlcF;         // element offset of the slice in a B row
                    tma_gather4(dst + (unsigned)(sl * kG4AtomBytes), &bmap, x, ca.x, cb.x, ca.y, cb.y, bar, pol_rows);
                    tma_gather4(dst + (unsigned)(sl * kG4AtomBytes + 512), &bmap, x, ca.z, cb.z, ca.w, cb.w, bar, pol_rows);
                }
            }
            bulk_copy_g2s_hint(vals_s + (unsigned)(st * kG4ValBytes), vals_base + (size_t)rf * kG4ValBytes,
                               (unsigned)kG4ValBytes, bar, pol_stream);
        }
    };

    const int g = lane >> 2, tid = lane & 3;

    int rf = 0;
#pragma unroll 1
    for (int i = 0; i < D - 1; ++i) {
        if (rf < nb) { fetch(rf); ++rf; }
    }

    const int lm_mat = lane >> 3;
    const int lm_srow = g4_row_of_k(lane & 7);                   // shared-memory row of this lane's ldmatrix row
    int rb = 0;
    bool failed = false;
    long long be_next = ((kMode == 2) ? (long long)__ldg(a.seg_bend + u_lo) : unit_begin<kMode>(a, u_lo + 1)) - B0;

#pragma unroll 1
    for (int u = u_lo; u < u_hi && !failed; ++u) {
        // a shared last window ends where the piece ends (segments are never shared)
        const int be = (kMode == 2) ? (int)be_next : min((int)be_next, nb);
        if (u + 1 < u_hi) {
            be_next = ((kMode == 2) ? (long long)__ldg(a.seg_bend + u + 1) : unit_begin<kMode>(a, u + 2)) - B0;
        }
        // destination rows of this unit (accumulator rows 2*tid and 2*tid+1)
        int dst_row_lo = -1, dst_row_hi = -1;
        float* cbase = a.C;
        const bool shared_head = head_partial && u == u_lo;
        const bool shared_tail = tail_partial && u == u_hi - 1;
        if (kMode != 2 && (shared_head || shared_tail)) {
            // partial tile: slot 2*gid for the unit this group entered through, 2*gid+1 for the one it leaves through
            cbase = a.scratch + (size_t)(2 * gid + (shared_head ? 0 : 1)) * kWindowRows * N;
            dst_row_lo = 2 * tid; dst_row_hi = dst_row_lo + 1;
        } else if (kMode == 0) {
            dst_row_lo = u * kWindowRows + 2 * tid; dst_row_hi = dst_row_lo + 1;
            if (dst_row_lo >= a.M) dst_row_lo = -1;
            if (dst_row_hi >= a.M) dst_row_hi = -1;
        } else if (kMode == 1) {
            dst_row_lo = __ldg(a.win_rows + (size_t)u * kWindowRows + 2 * tid);
            dst_row_hi = __ldg(a.win_rows + (size_t)u * kWindowRows + 2 * tid + 1);
        } else {
            const unsigned tag = (unsigned)__ldg(a.seg_window + u);
            const int w = (int)(tag & ~kSoleSegFlag);
            if (tag & kSoleSegFlag) {
                dst_row_lo = w * kWindowRows + 2 * tid; dst_row_hi = dst_row_lo + 1;
                if (dst_row_lo >= a.M) dst_row_lo = -1;
                if (dst_row_hi >= a.M) dst_row_hi = -1;
            } else {
                cbase = a.scratch + (size_t)__ldg(a.seg_scratch + u) * kWindowRows * N;
                dst_row_lo = 2 * tid; dst_row_hi = dst_row_lo + 1;
            }
        }

        float acc[S][kMT][4];
#pragma unroll
        for (int s = 0; s < S; ++s)
#pragma unroll
            for (int t = 0; t < kMT; ++t) { acc[s][t][0] = acc[s][t][1] = acc[s][t][2] = acc[s][t][3] = 0.f; }

#pragma unroll 1
        while (rb < be) {
            const int st0 = rb & (D - 1);
            if (!mbar_wait_warp_hint(bars_s + 8 * st0, (unsigned)((rb / D) & 1), kSpinLimit, wait_hint_ns)) { failed = true; break; }
            if (!kTF32 && rb + 1 < be) {
                // ---- two blocks: one m16n8k16 per 16-feature tile ----
                const int st1 = (rb + 1) & (D - 1);
                if (!mbar_wait_warp_hint(bars_s + 8 * st1, (unsigned)(((rb + 1) / D) & 1), kSpinLimit, wait_hint_ns)) { failed = true; break; }
                unsigned bf0, bf1;
                asm volatile("ld.shared.u32 %0, [%1];" : "=r"(bf0) : "r"(vals_s + (unsigned)(st0 * kG4ValBytes + lane * 4)));
                asm volatile("ld.shared.u32 %0, [%1];" : "=r"(bf1) : "r"(vals_s + (unsigned)(st1 * kG4ValBytes + lane * 4)));
                const unsigned row_base = atoms_s + (unsigned)((((lm_mat >> 1) ? st1 : st0) * S) * kG4AtomBytes + lm_srow * 128);
#pragma unroll
                for (int s = 0; s < S; ++s) {
                    if (s < s_valid) {                        // warp-uniform
#pragma unroll
                        for (int t = 0; t < kMT; ++t) {
                            const int chunk = t * 2 + (lm_mat & 1);
                            unsigned r0, r1, r2, r3;
                            asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                                         : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
                                         : "r"(row_base + (unsigned)(s * kG4AtomBytes + ((chunk ^ lm_srow) << 4))));
                            mma_f16_m16n8k16(acc[s][t], r0, r1, r2, r3, bf0, bf1);
                        }
                    }
                }
                __syncwarp();
                if (rf < nb) { fetch(rf); ++rf; }
                if (rf < nb) { fetch(rf); ++rf; }
                rb += 2;
            } else {
                if (!kTF32) {
                    unsigned bfrag;
                    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(bfrag) : "r"(vals_s + (unsigned)(st0 * kG4ValBytes + lane * 4)));
                    const unsigned row_base = atoms_s + (unsigned)((st0 * S) * kG4AtomBytes + lm_srow * 128);
#pragma unroll
                    for (int s = 0; s < S; ++s) {
                        if (s < s_valid) {
#pragma unroll
                            for (int tp = 0; tp < kMT / 2; ++tp) {
                                // matrices (m lo, m hi) of tile 2tp and of tile 2tp+1
                                const int chunk = tp * 4 + (lm_mat >> 1) * 2 + (lm_mat & 1);
                                unsigned r0, r1, r2, r3;
                                asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                                             : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
                                             : "r"(row_base + (unsigned)(s * kG4AtomBytes + ((chunk ^ lm_srow) << 4))));
                                mma_f16_m16n8k8(acc[s][tp * 2], r0, r1, bfrag);
                                mma_f16_m16n8k8(acc[s][tp * 2 + 1], r2, r3, bfrag);
                            }
                        }
                    }
                } else {
                    const __half* hv = reinterpret_cast<const __half*>(vals_sm + st0 * kG4ValBytes);
                    const int vslot = (g * 4 + (tid >> 1)) * 2 + (tid & 1);
                    const unsigned b0 = __float_as_uint(__half2float(hv[vslot]));
                    const unsigned b1 = __float_as_uint(__half2float(hv[vslot + 4]));
                    // k = tid sits in shared-memory row 2*tid, k = tid+4 in row 2*tid+1; the lane reads
                    // features 4g..4g+3 of the slice (16-byte chunk g, swizzled by the row index)
                    const unsigned char* at = atoms + (size_t)(st0 * S) * kG4AtomBytes;
                    const int row_lo = 2 * tid, row_hi = 2 * tid + 1;
#pragma unroll
                    for (int s = 0; s < S; ++s) {
                        if (s < s_valid) {
                            const float4 lo = *reinterpret_cast<const float4*>(at + s * kG4AtomBytes + row_lo * 128 + ((g ^ row_lo) << 4));
                            const float4 hi = *reinterpret_cast<const float4*>(at + s * kG4AtomBytes + row_hi * 128 + ((g ^ row_hi) << 4));
                            mma_tf32_m16n8k8(acc[s][0], to_tf32_rna(lo.x), to_tf32_rna(lo.y),
                                             to_tf32_rna(hi.x), to_tf32_rna(hi.y), b0, b1);
                            mma_tf32_m16n8k8(acc[s][1], to_tf32_rna(lo.z), to_tf32_rna(lo.w),
                                             to_tf32_rna(hi.z), to_tf32_rna(hi.w), b0, b1);
                        }
                    }
                }
                __syncwarp();
                if (rf < nb) { fetch(rf); ++rf; }
                rb += 1;
            }
        }
        if (failed) break;

        // ---- flush: acc[s][t] = {D[g][2tid], D[g][2tid+1], D[g+8][2tid], D[g+8][2tid+1]} ----
        if (kTF32) {
            // lane (g, tid) holds features 4g..4g+3 of the slice for window rows 2tid and 2tid+1
#pragma unroll
            for (int s = 0; s < S; ++s) {
                const int n = f0 + s * kSlcF + 4 * g;
                if (s < s_valid && n < N) {
                    if (dst_row_lo >= 0)
                        st_stream_float4(reinterpret_cast<float4*>(cbase + (size_t)dst_row_lo * N + n),
                                         make_float4(acc[s][0][0], acc[s][0][2], acc[s][1][0], acc[s][1][2]));
                    if (dst_row_hi >= 0)
                        st_stream_float4(reinterpret_cast<float4*>(cbase + (size_t)dst_row_hi * N + n),
                                         make_float4(acc[s][0][1], acc[s][0][3], acc[s][1][1], acc[s][1][3]));
                }
            }
        } else {
#pragma unroll
            for (int s = 0; s < S; ++s) {
                if (s < s_valid) {
#pragma unroll
                    for (int t = 0; t < kMT; ++t) {
                        const int n = f0 + s * kSlcF + t * 16 + g;
                        const bool c0 = n < N, c1 = n + 8 < N;   // padded operand columns are not stored
                        if (dst_row_lo >= 0) {
                            float* r = cbase + (size_t)dst_row_lo * N + n;
                            if (c0) st_stream_float(r, acc[s][t][0]);
                            if (c1) st_stream_float(r + 8, acc[s][t][2]);
                        }
                        if (dst_row_hi >= 0) {
                            float* r = cbase + (size_t)dst_row_hi * N + n;
                            if (c0) st_stream_float(r, acc[s][t][1]);
                            if (c1) st_stream_float(r + 8, acc[s][t][3]);
                        }
                    }
                }
            }
        }
    }
    if (failed) {
        if (lane == 0) atomicExch(status, kStatusFullTimeout);
        // collect the copies still in flight into this warp's ring before leaving
        for (int i = rb; i < rf; ++i) {
            if (!mbar_wait_warp(bars_s + 8 * (i & (D - 1)), (unsigned)((i / D) & 1), kSpinLimit)) break;
        }
    }
}

// Adds the partial tiles of every window that several groups shared, in block order, and writes the
// window's rows. One CTA per group; the CTA of the group in which a shared window begins owns it:
// its own tail slot comes first, then the head slots of the groups that follow, up to the group in
// which the window ends.
template <int kMode>
__global__ void __launch_bounds__(128)
g4_chain_merge_kernel(TileArgs a, int groups_total)
{
    const int g = blockIdx.x;
    const int2* shared_windows = reinterpret_cast<const int2*>(a.scratch + (size_t)2 * groups_total * kWindowRows * a.N);
    const int2 mine = shared_windows[g];
    const int unit = mine.y;
    if (unit < 0 || mine.x == unit) return;                      // no window begins here and continues in the next group
    int last = g + 1;                                            // groups g+1 .. last hold the rest of the window
    while (last + 1 < groups_total && shared_windows[last].y == unit) ++last;
    const int N = a.N;
    const size_t tile = (size_t)kWindowRows * N;
    for (int idx = threadIdx.x; idx < kWindowRows * N; idx += blockDim.x) {
        const int r = idx / N, col = idx - r * N;
        const int row = (kMode == 1) ? __ldg(a.win_rows + (size_t)unit * kWindowRows + r) : unit * kWindowRows + r;
        if (row < 0 || row >= a.M) continue;
        float acc = a.scratch[(size_t)(2 * g + 1) * tile + idx];
        for (int h = g + 1; h <= last; ++h) acc += a.scratch[(size_t)(2 * h) * tile + idx];
        a.C[(size_t)row * N + col] = acc;
    }
}

// ---- host side ------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_tiled_entry()
{
    static EncodeTiledFn fn = [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q = cudaDriverEntryPointSymbolNotFound;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
            q != cudaDriverEntryPointSuccess) p = nullptr;
        return reinterpret_cast<EncodeTiledFn>(p);
    }();
    return fn;
}

// Tensor map of the dense operand: rows of `ldb` elements, K rows, box = 128 bytes x 1 row.
static int make_b_map(CUtensorMap* map, const void* B, bool f32, long long K, int ldb)
{
    EncodeTiledFn enc = encode_tiled_entry();
    RA_REQUIRE(enc != nullptr, RA_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
    const int elem = f32 ? 4 : 2;
    const cuuint64_t gdim[2] = {(cuuint64_t)ldb, (cuuint64_t)K};
    const cuuint64_t gstride[1] = {(cuuint64_t)ldb * elem};
    const cuuint32_t box[2] = {(cuuint32_t)(128 / elem), 1u};
    const cuuint32_t estride[2] = {1u, 1u};
    const CUresult r = enc(map, f32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2,
                           const_cast<void*>(B), gdim, gstride, box, estride, CU_TENSOR_MAP_INTERLEAVE_NONE,
                           CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    RA_REQUIRE(r == CUDA_SUCCESS, RA_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d (ldb=%d, K=%lld)",
               (int)r, ldb, K);
    return RA_OK;
}

static int env_int(const char* name, int fallback)
{
    const char* e = std::getenv(name);
    return e ? std::atoi(e) : fallback;
}

// Launch shape of the ring for one SpMM: slices per warp, ring depth, CTA shape and the number of
// groups the work axis is cut into. One function so that the caller that sizes the scratch of the
// partial tiles and the launcher agree.
struct G4Config {
    bool ok = false;
    int slices_total = 0, S = 0, D = 0, wpg = 0, groups_per_cta = 0, warps = 0, ctas = 0, waves = 1;
    size_t smem = 0;
    long long groups = 0;
};

static G4Config g4_configure(bool tf32, int mode, const TileArgs& a)
{
    G4Config c;
    const int row_bytes = a.ldb * (tf32 ? 4 : 2);
    if (row_bytes % 16 != 0 || row_bytes > 2048 || row_bytes <= 0) return c;
    c.slices_total = (row_bytes + 127) / 128;
    // slices per warp and ring depth: measured defaults, RA_G4_SLICES / RA_G4_DEPTH override
    c.S = env_int("RA_G4_SLICES", 0);
    if (c.S != 1 && c.S != 2 && c.S != 4) c.S = (c.slices_total >= 4 && !tf32) ? 4 : (c.slices_total >= 2 ? 2 : 1);
    // Ring depth: 4 stages; 8 for the FP16 path with one slice per warp (N <= 64). That kernel holds 16
    // warps per SM by its registers whatever the ring costs, and with 1 KB stages four of them are too
    // few bytes in flight when the rows come from DRAM (configuration 5 at N=64: 3.1 vs 7.9 ms); with
    // wider slices 8 stages cost resident warps instead (35-150 % slower).
    c.D = env_int("RA_G4_DEPTH", 0);
    if (c.D != 2 && c.D != 4 && c.D != 8) c.D = (!tf32 && c.S == 1) ? 8 : 4;
    if (!tf32 && c.D < 4) c.D = 4;                  // the FP16 path consumes two stages at a time
    c.wpg = (c.slices_total + c.S - 1) / c.S;       // warps per group
    c.groups_per_cta = std::max(1, 4 / c.wpg);
    c.warps = c.wpg * c.groups_per_cta;
    c.smem = (size_t)c.warps * c.D * (c.S * kG4AtomBytes + kG4ValBytes + 8) + kG4AtomBytes;
    constexpr size_t kSmemCap = 227 * 1024;         // dynamic shared memory a CTA can have
    if (c.smem > kSmemCap || c.warps > 8) return c;
    const long long weight = a.total_blocks + a.num_units;
    const int ctas_per_sm = (int)std::max<size_t>(1, std::min<size_t>(16, (220 * 1024) / (c.smem + 1024)));
    // groups per resident slot: the FP16 path on windows (even unit lengths) is fastest with one
    // piece per resident group (C3 4.8 vs 5.1 ms); TF32 and the segment lists, whose pieces differ
    // more in cost, with three
    const int waves = std::max(1, env_int("RA_G4_WAVES", (!tf32 && mode != 2) ? 1 : 3));
    c.waves = waves;
    long long groups = (long long)sm_count() * ctas_per_sm * c.groups_per_cta * waves;
    groups = std::min(groups, std::max<long long>(1, weight / 48));
    c.ctas = (int)((groups + c.groups_per_cta - 1) / c.groups_per_cta);
    c.groups = (long long)c.ctas * c.groups_per_cta;
    c.ok = true;
    return c;
}

// Floats of scratch the window families need for the partial tiles of shared windows (two
// tiles of 8 x N per group); 0 when the ring does not apply to the shape.
long long tile_gather4_split_scratch_floats(bool tf32, int mode, const TileArgs& a)
{
    if (mode == 2 || env_int("RA_G4_SPLIT", 1) == 0) return 0;
    const G4Config c = g4_configure(tf32, mode, a);
    return c.ok ? 2ll * c.groups * kWindowRows * a.N + 2ll * c.groups : 0;   // partial tiles + one int2 per group
}

template <bool kTF32, int kMode, int S, int D>
static int launch_g4(const CUtensorMap& map, const TileArgs& a, const G4Config& cfg, cudaStream_t st, int* status)
{
    auto kern = tile_spmm_gather4_kernel<kTF32, kMode, S, D>;
    static std::atomic<unsigned long long> configured{0};
    RA_CUDA_TRY(configure_once_per_device(configured, [&]() {
        const size_t most = (size_t)8 * D * (S * kG4AtomBytes + kG4ValBytes + 8) + kG4AtomBytes;   // 8 warps
        return cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)std::min<size_t>(most, 227 * 1024));
    }));
    // g4_configure counts the CTAs an SM holds by shared memory; registers can allow fewer (the FP16
    // kernels use 126 per thread: 4 CTAs of 128 threads), and a grid of 5 CTAs per SM on 4 resident ones
    // runs a last quarter wave on its own. Size the grid by what is really resident.
    G4Config c = cfg;
    int resident = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&resident, kern, c.warps * 32, c.smem) == cudaSuccess && resident > 0) {
        const long long fit = (long long)sm_count() * resident * c.groups_per_cta * c.waves;
        if (fit < c.groups) {
            c.ctas = (int)((fit + c.groups_per_cta - 1) / c.groups_per_cta);
            c.groups = (long long)c.ctas * c.groups_per_cta;
        }
    }
    // Windows are shared between groups when the caller gave room for the partial tiles and whole
    // windows would leave the pieces uneven: the longest window is more than an eighth of a piece.
    // With many short windows per piece the groups keep whole windows: they then all start at a window
    // boundary and sweep the (sorted) columns of their windows at the same pace, which the L2 rewards
    // (configuration 3 TC_DIRECT on one GPU: 9.3 GB of DRAM reads against 21.3 GB with arbitrary cuts,
    // same time), and there is no merge launch.
    const long long piece = (a.total_blocks + a.num_units) / std::max<long long>(1, c.groups);
    const int split_env = env_int("RA_G4_SPLIT", 1);
    const bool uneven = split_env == 2 || ((long long)a.max_unit_blocks + 1) * 8 > piece;
    const bool split = kMode != 2 && split_env != 0 && uneven && a.scratch != nullptr &&
                       a.scratch_floats >= 2ll * c.groups * kWindowRows * a.N + 2ll * c.groups;
    kern<<<c.ctas, c.warps * 32, c.smem, st>>>(map, a, c.slices_total, c.wpg, (int)c.groups, status,
                                               (unsigned)std::max(0, env_int("RA_G4_WAIT_HINT_NS", 0)),
                                               env_int("RA_G4_L2POLICY", 1), split ? 1 : 0);
    RA_KERNEL_CHECK();
    if (split) {
        g4_chain_merge_kernel<(kMode == 2 ? 0 : kMode)><<<(unsigned)c.groups, 128, 0, st>>>(a, (int)c.groups);
        RA_KERNEL_CHECK();
    }
    return RA_OK;
}

// Runs the unit list of `a` with the TMA gather ring. B: fp32 (kTF32) or fp16 operand with rows of
// a.ldb elements; K rows. Returns RA_ERR_UNSUPPORTED when the shape does not fit (the caller
// then uses the cp.async ring).
template <bool kTF32, int kMode>
int launch_tile_gather4(const TileArgs& a, const void* B, long long K, cudaStream_t st, int* status)
{
    if (!aligned16(B) || K <= 0 || K >= (1ll << 31)) return RA_ERR_UNSUPPORTED;
    const G4Config c = g4_configure(kTF32, kMode, a);
    if (!c.ok) return RA_ERR_UNSUPPORTED;
    CUtensorMap map;
    const int rc = make_b_map(&map, B, kTF32, K, a.ldb);
    if (rc != RA_OK) return rc;
#define RA_G4_CASE(SS, DD) if (c.S == SS && c.D == DD) return launch_g4<kTF32, kMode, SS, DD>(map, a, c, st, status)
    RA_G4_CASE(1, 2); RA_G4_CASE(1, 4); RA_G4_CASE(1, 8); RA_G4_CASE(2, 2); RA_G4_CASE(2, 4); RA_G4_CASE(2, 8);
    RA_G4_CASE(4, 2); RA_G4_CASE(4, 4); RA_G4_CASE(4, 8);
#undef RA_G4_CASE
    return RA_ERR_UNSUPPORTED;
}

template int launch_tile_gather4<false, 0>(const TileArgs&, const void*, long long, cudaStream_t, int*);
template int launch_tile_gather4<false, 1>(const TileArgs&, const void*, long long, cudaStream_t, int*);
template int launch_tile_gather4<false, 2>(const TileArgs&, const void*, long long, cudaStream_t, int*);
template int launch_tile_gather4<true, 0>(const TileArgs&, const void*, long long, cudaStream_t, int*);
template int launch_tile_gather4<true, 1>(const TileArgs&, const void*, long long, cudaStream_t, int*);
template int launch_tile_gather4<true, 2>(const TileArgs&, const void*, long long, cudaStream_t, int*);

}  // namespace ra
