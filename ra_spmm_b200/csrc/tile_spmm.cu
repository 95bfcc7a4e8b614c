// Tile SpMM kernels for sm_100a: TC_DIRECT, COMMUNITY_TC and SEGMENT_HYBRID on
// the FP16 and TF32 paths.
//
// Replace run_ra_tc_direct_plan[_tf32] (tc/ra_tc_direct.cu:805-894),
// run_ra_community_tc_plan[_tf32] (tc/ra_community_tc.cu:476-552) and
// run_ra_segment_hybrid_plan[_tf32] (tc/ra_segment_hybrid.cu:548-668) with
// their kernels. Numerics are those of the reference: per 8-vector block one
// m16n8k8 tensor-core MMA with the gathered dense tile as the A operand and
// the packed sparse 8x8 block as the B operand, fp32 accumulation in block
// order; FP16 path = B rounded to fp16 (RNE), TF32 path = B rounded with
// cvt.rna.tf32, sparse values widened from fp16.
//
// Execution model (differs from the reference's one-CTA-per-window grid):
//   * a "unit" is a window (TC_DIRECT, COMMUNITY_TC) or a <=64-block segment
//     (SEGMENT_HYBRID); the blocks of consecutive units are contiguous in
//     memory, so a warp streams one long block range and flushes its
//     accumulators at unit boundaries;
//   * the unit list is cut into weight-balanced contiguous ranges (weight =
//     blocks + 1 per unit) and a persistent grid of warp groups takes one
//     range each; a group has one warp per 128-byte column slice of B
//     (64 fp16 or 32 fp32 features), so warps never synchronise with each
//     other;
//   * each warp runs its own shared-memory ring (8 stages on the FP16 path, 4 on
//     the TF32 path, whose stages are twice as large): per block it issues
//     16-byte cp.async copies of its slice of the 8 gathered B rows plus the
//     128-byte packed sparse block, and consumes stages with ldmatrix.trans
//     (fp16) or conflict-free 32-bit loads (tf32). The ring runs ahead across
//     unit boundaries, so short windows do not drain the pipeline.
//   * gather indices (atox) are prefetched four blocks per coalesced load.
#include "tile_common.cuh"

#include <algorithm>
#include <cstdlib>

namespace ra {

constexpr int kStages      = 8;     // ring depth of the FP16 path (and of the bulk-copy variant)
// Ring depth of the per-warp kernel (template parameter kDepth): 8 stages, or 4 stages and twice
// the resident warps. Measured on B200: the FP16 path is faster with 8 everywhere (C3 7.8 vs 8.5 ms);
// the TF32 path, whose stages are twice as large, is faster with 4 at N = 256 (C3 17.3 vs 21.5 ms)
// and on SEGMENT_HYBRID (C4 5.4 vs 6.1 ms, C2 1.20 vs 1.30 ms), slower with 4 on TC_DIRECT /
// COMMUNITY_TC at N <= 128 (C2 1.6 vs 1.3 ms).
constexpr int kRowBytesF16 = 128 + 16;   // 64 halves + pad: ldmatrix rows hit distinct banks
constexpr int kRowBytesF32 = 128 + 32;   // 32 floats + pad: (8k + g) mod 32 distinct
constexpr int kStageF16    = 8 * kRowBytesF16 + 128;   // + packed sparse block
constexpr int kStageF32    = 8 * kRowBytesF32 + 128;

// kMode: 0 natural windows, 1 window-row table (COMMUNITY_TC), 2 segments.
// kMT: 16-feature tiles per warp slice (4 for fp16, 2 for tf32).
// FP16: two consecutive blocks of a unit feed one m16n8k16 MMA (k 0-7 from the
// first block's stage, k 8-15 from the second's); an odd last block uses m16n8k8.
// kZC: the packed sparse block of a stage is decoded from the zero-compressed arrays (each lane
// fetches its own two fragment halves; the loads of block i are issued when block i is fetched
// and stored to the stage one fetch later, so their latency stays off the critical path).
template <bool kTF32, int kMode, bool kZC, int kDepth>
__global__ void __launch_bounds__(256)
tile_spmm_kernel(TileArgs a, const void* __restrict__ Bmat, int slices, int groups_total)
{
    constexpr int kMT       = kTF32 ? 2 : 4;
    constexpr int kRowBytes = kTF32 ? kRowBytesF32 : kRowBytesF16;
    constexpr int kStage    = kTF32 ? kStageF32 : kStageF16;
    constexpr int kElem     = kTF32 ? 4 : 2;
    constexpr int kSliceF   = 128 / kElem;          // features per slice
    constexpr int kRingStages = kDepth;
    static_assert(kDepth == 4 || kDepth == 8, "ring depth");
    extern __shared__ __align__(16) unsigned char smem[];

    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    const int groups_per_cta = (blockDim.x >> 5) / slices;
    const int grp = warp / slices;
    if (grp >= groups_per_cta) return;
    const int slice = warp - grp * slices;
    const int gid = blockIdx.x * groups_per_cta + grp;
    if (gid >= groups_total) return;

    // ---- this group's contiguous unit range, balanced by blocks + units ----
    const long long total_w = a.total_blocks + a.num_units;
    const int u_lo = unit_lower_bound<kMode>(a, total_w * gid / groups_total);
    const int u_hi = unit_lower_bound<kMode>(a, total_w * (gid + 1) / groups_total);
    if (u_lo >= u_hi) return;
    const long long B0 = unit_begin<kMode>(a, u_lo);
    const int nb = (int)(unit_begin<kMode>(a, u_hi) - B0);      // blocks of this range

    unsigned char* ring = smem + (size_t)warp * kRingStages * kStage;
    const unsigned ring_s = (unsigned)__cvta_generic_to_shared(ring);
    const int N = a.N;
    const int ldb = a.ldb;                                   // multiple of 16, >= N
    const int f0 = slice * kSliceF;                          // first feature of the slice
    const int mt_valid = min(kMT, (ldb - f0 + 15) >> 4);
    const size_t row_bytes_g = (size_t)ldb * kElem;

    // ---- per-lane constants of the gather: lane copies chunk `ch` of rows `row`, `row+4`
    const int row = lane >> 3, ch = lane & 7;
    const bool chunk_ok = (f0 + ch * (16 / kElem)) < ldb;
    const unsigned char* b_lane = static_cast<const unsigned char*>(Bmat) + (size_t)(f0 * kElem + ch * 16);
    const unsigned dst_lo = row * kRowBytes + ch * 16;
    const unsigned dst_hi = dst_lo + 4 * kRowBytes;
    const unsigned char* vals_lane = reinterpret_cast<const unsigned char*>(a.vals) + (size_t)B0 * 128 + lane * 16;
    const int* atox_base = a.atox + B0 * kVecPerBlock;
    const int atox_len = nb * kVecPerBlock;

    // ---- gather-index prefetch: 4 blocks (32 indices) per register ----
    int ab = 0;                                              // first block (relative) held by ax
    auto load_ax = [&](int blk) -> int {
        const int idx = blk * kVecPerBlock + lane;
        return (idx < atox_len) ? __ldg(atox_base + idx) : 0;
    };
    int ax = load_ax(0), ax_next = load_ax(4);

    // ---- zero-compressed values: decode pipeline held in registers ----
    unsigned long long zc_mask = 0ull;                       // mask / base of the next block to fetch
    int zc_base = 0;
    unsigned zc_h0 = 0u, zc_h1 = 0u;                         // halves of block zc_pending, loads in flight
    int zc_pending = -1;
    if (kZC && nb > 0) {
        zc_mask = __ldg(a.val_masks + B0);
        zc_base = __ldg(a.val_base + B0);
    }
    auto zc_flush = [&]() {                                  // store the pending fragment word to its stage
        if (zc_pending >= 0) {
            const unsigned dst = ring_s + (unsigned)((zc_pending & (kRingStages - 1)) * kStage) + 8 * kRowBytes + lane * 4;
            asm volatile("st.shared.u32 [%0], %1;" :: "r"(dst), "r"(zc_h0 | (zc_h1 << 16)) : "memory");
            zc_pending = -1;
        }
    };

    auto fetch = [&](int rf) {                               // rf: block index relative to B0
        if (rf >= ab + 4) { ax = ax_next; ab += 4; ax_next = load_ax(ab + 4); }
        const unsigned st = ring_s + (unsigned)((rf & (kRingStages - 1)) * kStage);
        const int sub = (rf - ab) * 8 + row;
        const int c_lo = __shfl_sync(0xffffffffu, ax, sub);
        const int c_hi = __shfl_sync(0xffffffffu, ax, sub + 4);
        if (chunk_ok) {
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" :: "r"(st + dst_lo), "l"(b_lane + (size_t)c_lo * row_bytes_g) : "memory");
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" :: "r"(st + dst_hi), "l"(b_lane + (size_t)c_hi * row_bytes_g) : "memory");
        }
        if (kZC) {
            zc_flush();                                        // block rf-1: its loads had one fetch interval
            const unsigned long long m = zc_mask;
            const int base = zc_base;
            if (rf + 1 < nb) {                                 // mask/base of the next block
                zc_mask = __ldg(a.val_masks + B0 + rf + 1);
                zc_base = __ldg(a.val_base + B0 + rf + 1);
            }
            // fragment word of lane (g, tid): halves (row g, vector 2tid) and (row g, vector 2tid+1)
            zc_h0 = zc_value_bits(m, base, a.vals_zc, 2 * (lane & 3), lane >> 2);
            zc_h1 = zc_value_bits(m, base, a.vals_zc, 2 * (lane & 3) + 1, lane >> 2);
            zc_pending = rf;
        } else if (lane < 8) {
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" :: "r"(st + 8 * kRowBytes + lane * 16), "l"(vals_lane + (size_t)rf * 128) : "memory");
        }
    };

    int rf = 0;
#pragma unroll 1
    for (int i = 0; i < kRingStages - 1; ++i) {
        if (rf < nb) { fetch(rf); ++rf; }
        cp_async_commit();
    }
    if (kZC && rf >= nb) zc_flush();                           // short range: nothing more will be fetched

    const int g = lane >> 2, tid = lane & 3;
    // ldmatrix lane roles: matrix = lane>>3 -> (k half = mat>>1, m half = mat&1), row in matrix = lane&7
    const int lm_mat = lane >> 3, lm_row = lane & 7;
    int rb = 0;
    long long be_next = ((kMode == 2) ? (long long)__ldg(a.seg_bend + u_lo) : unit_begin<kMode>(a, u_lo + 1)) - B0;

#pragma unroll 1
    for (int u = u_lo; u < u_hi; ++u) {
        const int be = (int)be_next;
        if (u + 1 < u_hi) {
            be_next = ((kMode == 2) ? (long long)__ldg(a.seg_bend + u + 1) : unit_begin<kMode>(a, u + 2)) - B0;
        }
        // destination rows of this unit
        int dst_row_lo = -1, dst_row_hi = -1;         // rows for accumulator rows 2*tid, 2*tid+1
        float* base = a.C;
        if (kMode == 0) {
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
                base = a.scratch + (size_t)__ldg(a.seg_scratch + u) * kWindowRows * N;
                dst_row_lo = 2 * tid; dst_row_hi = dst_row_lo + 1;
            }
        }

        float acc[kMT][4];
#pragma unroll
        for (int t = 0; t < kMT; ++t) { acc[t][0] = acc[t][1] = acc[t][2] = acc[t][3] = 0.f; }

#pragma unroll 1
        while (rb < be) {
            if (!kTF32 && rb + 1 < be) {
                // ---- two blocks: one m16n8k16 per 16-feature tile ----
                cp_async_wait<kRingStages - 3>();
                __syncwarp();
                const unsigned s0 = ring_s + (unsigned)((rb & (kRingStages - 1)) * kStage);
                const unsigned s1 = ring_s + (unsigned)(((rb + 1) & (kRingStages - 1)) * kStage);
                unsigned bf0, bf1;
                asm volatile("ld.shared.u32 %0, [%1];" : "=r"(bf0) : "r"(s0 + 8 * kRowBytes + lane * 4));
                asm volatile("ld.shared.u32 %0, [%1];" : "=r"(bf1) : "r"(s1 + 8 * kRowBytes + lane * 4));
                const unsigned lm_addr = ((lm_mat >> 1) ? s1 : s0) + lm_row * kRowBytes + (lm_mat & 1) * 16;
#pragma unroll
                for (int t = 0; t < kMT; ++t) {
                    if (t < mt_valid) {                       // warp-uniform
                        unsigned r0, r1, r2, r3;
                        asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                                     : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(lm_addr + t * 32));
                        mma_f16_m16n8k16(acc[t], r0, r1, r2, r3, bf0, bf1);
                    }
                }
                __syncwarp();
                if (rf < nb) { fetch(rf); ++rf; } else if (kZC) zc_flush();
                cp_async_commit();
                if (rf < nb) { fetch(rf); ++rf; } else if (kZC) zc_flush();
                cp_async_commit();
                rb += 2;
            } else {
                cp_async_wait<kRingStages - 2>();
                __syncwarp();
                const unsigned char* st = ring + (size_t)(rb & (kRingStages - 1)) * kStage;
                const unsigned char* sv = st + 8 * kRowBytes;
                if (!kTF32) {
                    const unsigned bfrag = *reinterpret_cast<const unsigned*>(sv + lane * 4);
                    const unsigned s0 = ring_s + (unsigned)((rb & (kRingStages - 1)) * kStage);
                    // x4.trans over one stage: matrices (m lo, m hi) of tile 2tp and of tile 2tp+1
                    const unsigned lm1 = s0 + lm_row * kRowBytes + (lm_mat & 1) * 16 + (lm_mat >> 1) * 32;
#pragma unroll
                    for (int tp = 0; tp < kMT / 2; ++tp) {
                        if (tp * 2 < mt_valid) {
                            // a tile beyond mt_valid still reads inside the stage row (unused result)
                            unsigned r0, r1, r2, r3;
                            asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                                         : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(lm1 + tp * 64));
                            mma_f16_m16n8k8(acc[tp * 2], r0, r1, bfrag);
                            if (tp * 2 + 1 < mt_valid) mma_f16_m16n8k8(acc[tp * 2 + 1], r2, r3, bfrag);
                        }
                    }
                } else {
                    const __half* hv = reinterpret_cast<const __half*>(sv);
                    const int vslot = (g * 4 + (tid >> 1)) * 2 + (tid & 1);
                    const unsigned b0 = __float_as_uint(__half2float(hv[vslot]));
                    const unsigned b1 = __float_as_uint(__half2float(hv[vslot + 4]));
                    // MMA row <-> feature map chosen so that a lane's operands are contiguous: tile 0
                    // rows (g, g+8) = features (4g, 4g+1), tile 1 rows (g, g+8) = (4g+2, 4g+3): one
                    // 128-bit load per gathered row instead of four 32-bit ones, and 128-bit stores.
                    // Features past the operand width (last slice) multiply stale shared memory;
                    // their rows are never stored.
                    const float4 lo = *reinterpret_cast<const float4*>(st + tid * kRowBytes + g * 16);
                    const float4 hi = *reinterpret_cast<const float4*>(st + (tid + 4) * kRowBytes + g * 16);
                    mma_tf32_m16n8k8(acc[0], to_tf32_rna(lo.x), to_tf32_rna(lo.y),
                                     to_tf32_rna(hi.x), to_tf32_rna(hi.y), b0, b1);
                    mma_tf32_m16n8k8(acc[kMT - 1], to_tf32_rna(lo.z), to_tf32_rna(lo.w),
                                     to_tf32_rna(hi.z), to_tf32_rna(hi.w), b0, b1);
                }
                __syncwarp();
                if (rf < nb) { fetch(rf); ++rf; } else if (kZC) zc_flush();
                cp_async_commit();
                rb += 1;
            }
        }

        // flush: acc[t] = {D[g][2tid], D[g][2tid+1], D[g+8][2tid], D[g+8][2tid+1]},
        // D[feature][window row]
        if (kTF32) {
            // lane (g, tid) holds features f0 + 4g .. +3 of window rows 2tid and 2tid+1
            const int n = f0 + 4 * g;
            if (n < N) {
                if (dst_row_lo >= 0)
                    *reinterpret_cast<float4*>(base + (size_t)dst_row_lo * N + n) =
                        make_float4(acc[0][0], acc[0][2], acc[kMT - 1][0], acc[kMT - 1][2]);
                if (dst_row_hi >= 0)
                    *reinterpret_cast<float4*>(base + (size_t)dst_row_hi * N + n) =
                        make_float4(acc[0][1], acc[0][3], acc[kMT - 1][1], acc[kMT - 1][3]);
            }
        } else
#pragma unroll
        for (int t = 0; t < kMT; ++t) {
            if (t < mt_valid) {
                const int n = f0 + t * 16 + g;
                const bool c0 = n < N, c1 = n + 8 < N;       // padded operand columns are not stored
                if (dst_row_lo >= 0) {
                    float* r = base + (size_t)dst_row_lo * N + n;
                    if (c0) r[0] = acc[t][0];
                    if (c1) r[8] = acc[t][2];
                }
                if (dst_row_hi >= 0) {
                    float* r = base + (size_t)dst_row_hi * N + n;
                    if (c0) r[0] = acc[t][1];
                    if (c1) r[8] = acc[t][3];
                }
            }
        }
    }
    cp_async_wait<0>();
}

// ---------------------------------------------------------------------------
// TMA variant of the staged kernel: the gathered B rows and the packed sparse
// block of a stage arrive by bulk asynchronous copies (cp.async.bulk, one copy
// per whole B row, issued by one lane each of the group's first warp) and are
// tracked by an mbarrier per stage ("full": transaction bytes; "empty": one
// arrival per consumer warp). The warps of a group share the ring; each warp
// still multiplies its own 128-byte column slice. Every wait is bounded: after
// kSpinLimit polls the warp records an error code in the status word and returns.
// ---------------------------------------------------------------------------

template <bool kTF32, int kMode>
__global__ void __launch_bounds__(256)
tile_spmm_tma_kernel(TileArgs a, const void* __restrict__ Bmat, int slices, int groups_total,
                     int group_bytes, int* __restrict__ status, int full_poll_limit)
{
    constexpr int kMT     = kTF32 ? 2 : 4;
    constexpr int kElem   = kTF32 ? 4 : 2;
    constexpr int kSliceF = 128 / kElem;
    constexpr int kPad    = kTF32 ? 32 : 16;
    extern __shared__ __align__(128) unsigned char smem[];

    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    const int groups_per_cta = (blockDim.x >> 5) / slices;
    const int grp = warp / slices;
    const int slice = warp - grp * slices;
    const int gid = blockIdx.x * groups_per_cta + grp;
    const bool has_group = grp < groups_per_cta && gid < groups_total;
    const int N = a.N;
    const int row_bytes = N * kElem;                     // one gathered B row
    const int row_stride = row_bytes + kPad;
    const int stage_bytes = 8 * row_stride + 128;

    unsigned char* gbase = smem + (size_t)grp * group_bytes;
    const unsigned gbase_s = (unsigned)__cvta_generic_to_shared(gbase);
    const unsigned full0 = gbase_s, empty0 = gbase_s + 8 * kStages;      // 8-byte barriers
    const unsigned ring_s = gbase_s + 128;
    unsigned char* ring = gbase + 128;

    if (has_group && slice == 0 && lane == 0) {
        for (int s = 0; s < kStages; ++s) { mbar_init(full0 + 8 * s, 1); mbar_init(empty0 + 8 * s, slices); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    if (!has_group) return;

    const long long total_w = a.total_blocks + a.num_units;
    const int u_lo = unit_lower_bound<kMode>(a, total_w * gid / groups_total);
    const int u_hi = unit_lower_bound<kMode>(a, total_w * (gid + 1) / groups_total);
    if (u_lo >= u_hi) return;
    const long long B0 = unit_begin<kMode>(a, u_lo);
    const int nb = (int)(unit_begin<kMode>(a, u_hi) - B0);

    const int f0 = slice * kSliceF;
    const int mt_valid = min(kMT, (N - f0 + 15) >> 4);
    const unsigned char* Bbytes = static_cast<const unsigned char*>(Bmat);
    const unsigned char* vals_base = reinterpret_cast<const unsigned char*>(a.vals) + (size_t)B0 * 128;
    const int* atox_base = a.atox + B0 * kVecPerBlock;
    const int atox_len = nb * kVecPerBlock;
    const bool producer = slice == 0;

    int ab = 0;
    auto load_ax = [&](int blk) -> int {
        const int idx = blk * kVecPerBlock + lane;
        return (idx < atox_len) ? __ldg(atox_base + idx) : 0;
    };
    int ax = 0, ax_next = 0;
    if (producer) { ax = load_ax(0); ax_next = load_ax(4); }
    bool failed = false;

    // producer warp: block rf -> stage rf % kStages; false = the stage was never released (nothing issued)
    auto fetch = [&](int rf) -> bool {
        if (rf >= ab + 4) { ax = ax_next; ab += 4; ax_next = load_ax(ab + 4); }
        const int st = rf & (kStages - 1);
        if (rf >= kStages) {                                  // wait until every warp released the stage
            if (!mbar_wait_warp(empty0 + 8 * st, (unsigned)(((rf >> 3) - 1) & 1), kSpinLimit)) { failed = true; return false; }
        }
        const int oct = (rf - ab) * 8;                        // lanes oct..oct+7 hold this block's columns
        const unsigned stage_s = ring_s + (unsigned)(st * stage_bytes);
        if (lane == oct) mbar_expect_tx(full0 + 8 * st, (unsigned)(8 * row_bytes + 128));
        __syncwarp();
        if (lane >= oct && lane < oct + 8) {
            bulk_copy_g2s(stage_s + (unsigned)((lane - oct) * row_stride),
                          Bbytes + (size_t)ax * (size_t)row_bytes, (unsigned)row_bytes, full0 + 8 * st);
        } else if (lane == ((oct + 8) & 31)) {
            bulk_copy_g2s(stage_s + (unsigned)(8 * row_stride), vals_base + (size_t)rf * 128, 128u, full0 + 8 * st);
        }
        return true;
    };

    int rf = 0;
    if (producer) {
#pragma unroll 1
        for (int i = 0; i < kStages - 1; ++i) {
            if (rf < nb && fetch(rf)) ++rf;
        }
    }

    const int g = lane >> 2, tid = lane & 3;
    const int lm_mat = lane >> 3, lm_row = lane & 7;
    int rb = 0;
    long long be_next = ((kMode == 2) ? (long long)__ldg(a.seg_bend + u_lo) : unit_begin<kMode>(a, u_lo + 1)) - B0;

#pragma unroll 1
    for (int u = u_lo; u < u_hi && !failed; ++u) {
        const int be = (int)be_next;
        if (u + 1 < u_hi) {
            be_next = ((kMode == 2) ? (long long)__ldg(a.seg_bend + u + 1) : unit_begin<kMode>(a, u + 2)) - B0;
        }
        int dst_row_lo = -1, dst_row_hi = -1;
        float* base = a.C;
        if (kMode == 0) {
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
                base = a.scratch + (size_t)__ldg(a.seg_scratch + u) * kWindowRows * N;
                dst_row_lo = 2 * tid; dst_row_hi = dst_row_lo + 1;
            }
        }
        float acc[kMT][4];
#pragma unroll
        for (int t = 0; t < kMT; ++t) { acc[t][0] = acc[t][1] = acc[t][2] = acc[t][3] = 0.f; }

#pragma unroll 1
        while (rb < be) {
            const int st0 = rb & (kStages - 1);
            const unsigned s0 = ring_s + (unsigned)(st0 * stage_bytes);
            if (!mbar_wait_warp(full0 + 8 * st0, (unsigned)((rb >> 3) & 1), full_poll_limit)) { failed = true; break; }
            if (!kTF32 && rb + 1 < be) {
                const int st1 = (rb + 1) & (kStages - 1);
                const unsigned s1 = ring_s + (unsigned)(st1 * stage_bytes);
                if (!mbar_wait_warp(full0 + 8 * st1, (unsigned)(((rb + 1) >> 3) & 1), full_poll_limit)) { failed = true; break; }
                unsigned bf0, bf1;
                asm volatile("ld.shared.u32 %0, [%1];" : "=r"(bf0) : "r"(s0 + 8 * row_stride + lane * 4));
                asm volatile("ld.shared.u32 %0, [%1];" : "=r"(bf1) : "r"(s1 + 8 * row_stride + lane * 4));
                const unsigned lm_addr = ((lm_mat >> 1) ? s1 : s0) + lm_row * row_stride + f0 * 2 + (lm_mat & 1) * 16;
#pragma unroll
                for (int t = 0; t < kMT; ++t) {
                    if (t < mt_valid) {
                        unsigned r0, r1, r2, r3;
                        asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                                     : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(lm_addr + t * 32));
                        mma_f16_m16n8k16(acc[t], r0, r1, r2, r3, bf0, bf1);
                    }
                }
                __syncwarp();
                if (lane == 0) { mbar_arrive(empty0 + 8 * st0); mbar_arrive(empty0 + 8 * st1); }
                if (producer) {
                    if (rf < nb && fetch(rf)) ++rf;
                    if (rf < nb && !failed && fetch(rf)) ++rf;
                }
                rb += 2;
            } else {
                if (!kTF32) {
                    unsigned bfrag;
                    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(bfrag) : "r"(s0 + 8 * row_stride + lane * 4));
                    const unsigned lm1 = s0 + lm_row * row_stride + f0 * 2 + (lm_mat & 1) * 16 + (lm_mat >> 1) * 32;
#pragma unroll
                    for (int tp = 0; tp < kMT / 2; ++tp) {
                        if (tp * 2 < mt_valid) {
                            unsigned r0, r1, r2, r3;
                            asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                                         : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(lm1 + tp * 64));
                            mma_f16_m16n8k8(acc[tp * 2], r0, r1, bfrag);
                            if (tp * 2 + 1 < mt_valid) mma_f16_m16n8k8(acc[tp * 2 + 1], r2, r3, bfrag);
                        }
                    }
                } else {
                    const unsigned char* stp = ring + (size_t)st0 * stage_bytes;
                    const __half* hv = reinterpret_cast<const __half*>(stp + 8 * row_stride);
                    const int vslot = (g * 4 + (tid >> 1)) * 2 + (tid & 1);
                    const unsigned b0 = __float_as_uint(__half2float(hv[vslot]));
                    const unsigned b1 = __float_as_uint(__half2float(hv[vslot + 4]));
#pragma unroll
                    for (int t = 0; t < kMT; ++t) {
                        if (t < mt_valid) {
                            const float* r_lo = reinterpret_cast<const float*>(stp + tid * row_stride) + f0 + t * 16 + g;
                            const float* r_hi = reinterpret_cast<const float*>(stp + (tid + 4) * row_stride) + f0 + t * 16 + g;
                            mma_tf32_m16n8k8(acc[t], to_tf32_rna(r_lo[0]), to_tf32_rna(r_lo[8]),
                                             to_tf32_rna(r_hi[0]), to_tf32_rna(r_hi[8]), b0, b1);
                        }
                    }
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(empty0 + 8 * st0);
                if (producer && rf < nb && fetch(rf)) ++rf;
                rb += 1;
            }
            if (failed) break;
        }
        if (failed) break;
#pragma unroll
        for (int t = 0; t < kMT; ++t) {
            if (t < mt_valid) {
                const int n = f0 + t * 16 + g;
                if (dst_row_lo >= 0) {
                    float* r = base + (size_t)dst_row_lo * N + n;
                    r[0] = acc[t][0]; r[8] = acc[t][2];
                }
                if (dst_row_hi >= 0) {
                    float* r = base + (size_t)dst_row_hi * N + n;
                    r[0] = acc[t][1]; r[8] = acc[t][3];
                }
            }
        }
    }
    if (failed) {
        if (lane == 0) atomicExch(status, kStatusFullTimeout);
        // A warp that gave up still owns the bulk copies it issued: the producer waits, under the
        // normal limit, until every stage it filled and nobody consumed has landed, so no copy is
        // in flight into this CTA's shared memory when the CTA ends.
        if (producer) {
            for (int i = rb; i < rf; ++i) {
                if (!mbar_wait_warp(full0 + 8 * (i & (kStages - 1)), (unsigned)((i >> 3) & 1), kSpinLimit)) break;
            }
        }
    }
}

// ---------------------------------------------------------------------------
// tcgen05 variant of the FP16 path: the packed sparse blocks go through the
// 5th-generation tensor cores with the accumulators in tensor memory.
//
//   D[128 features x 16] (TMEM, fp32) += A[128 x 16] * B[16 x 16]^T      per K-step (= 2 blocks)
//
//   A = the 16 gathered B rows of the two blocks, 128 features wide: an MN-major operand in
//       the 128-byte-swizzle canonical layout - atoms of [8 k-rows][64 features] (1 KB, 16-byte
//       chunk index XOR k-row), atom stride 1 KB along the features (LBO) and 2 KB along k (SBO).
//       The gather writes this layout directly with 16-byte cp.async.
//   B = the two packed 8x8 fp16 blocks exactly as the plan stores them: index r*8 + k is a K-major
//       core matrix (8 window rows x 16 bytes), so the 128-byte blocks are copied verbatim (LBO =
//       128 between the two blocks); MMA rows 8..15 read a zero region at +256 (SBO).
//   One thread issues tcgen05.mma per 128-feature panel and tcgen05.commit to the stage's
//   mbarrier; the stage is refilled after that barrier completes. At the end of a unit the four
//   warps read their 32 TMEM lanes (tcgen05.ld 32x32b) - lane = feature, column = window row -
//   and store 128-byte coalesced row segments of C.
// All waits are bounded; a timeout is reduced over the CTA at the next barrier, recorded in the
// status word, and the CTA frees its TMEM and returns.
// ---------------------------------------------------------------------------
constexpr int kTcStages = 4;
constexpr int kTcThreads = 128;
enum { kStatusMmaTimeout = 3 };

__device__ __forceinline__ unsigned long long tc5_smem_desc(unsigned saddr, unsigned lbo, unsigned sbo, unsigned layout) {
    unsigned long long d = 0;
    d |= (unsigned long long)((saddr >> 4) & 0x3FFFu);
    d |= (unsigned long long)((lbo >> 4) & 0x3FFFu) << 16;
    d |= (unsigned long long)((sbo >> 4) & 0x3FFFu) << 32;
    d |= 1ull << 46;                               // descriptor version of sm_100
    d |= (unsigned long long)(layout & 7u) << 61;  // 0 = no swizzle, 2 = 128-byte swizzle
    return d;
}

template <int kMode>
__device__ __forceinline__ void tc5_unit_bounds(const TileArgs& a, int u, long long B0, int& b, int& e) {
    if (kMode == 2) { b = (int)(__ldg(a.seg_bbegin + u) - B0); e = (int)(__ldg(a.seg_bend + u) - B0); }
    else { b = (int)(__ldg(a.block_offsets + u) - B0); e = (int)(__ldg(a.block_offsets + u + 1) - B0); }
}

template <int kMode>
__global__ void __launch_bounds__(kTcThreads)
tile_spmm_tc5_kernel(TileArgs a, const __half* __restrict__ Bh, int groups_total, int panels,
                     int* __restrict__ status)
{
    extern __shared__ unsigned char smem_raw[];
    __shared__ unsigned long long mma_done[kTcStages];
    __shared__ unsigned tmem_slot;
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    const unsigned smem_s = (unsigned)__cvta_generic_to_shared(smem);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int N = a.N;
    const int stage_bytes = panels * 4096 + 1024;            // A panels | 256 B blocks + 256 B zeros | pad
    const int tmem_cols = 64;                                // 4 / 2 / 1 units side by side for 1 / 2 / 4 panels

    // zero everything once: feature chunks beyond N and the B zero rows stay zero for good
    for (int i = tid; i < kTcStages * stage_bytes / 16; i += kTcThreads)
        reinterpret_cast<uint4*>(smem)[i] = make_uint4(0, 0, 0, 0);
    const unsigned bar0 = (unsigned)__cvta_generic_to_shared(&mma_done[0]);
    if (tid == 0) {
        for (int s = 0; s < kTcStages; ++s) mbar_init(bar0 + 8 * s, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) {
        const unsigned slot = (unsigned)__cvta_generic_to_shared(&tmem_slot);
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], 64;" :: "r"(slot) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const unsigned tmem = tmem_slot;

    // ---- unit range of this CTA ----
    const int gid = blockIdx.x;
    const long long total_w = a.total_blocks + a.num_units;
    int u_lo = 0, u_hi = 0;
    if (gid < groups_total) {
        u_lo = unit_lower_bound<kMode>(a, total_w * gid / groups_total);
        u_hi = unit_lower_bound<kMode>(a, total_w * (gid + 1) / groups_total);
    }
    const long long B0 = (u_lo < u_hi) ? unit_begin<kMode>(a, u_lo) : 0;
    const int* atox_base = a.atox + B0 * kVecPerBlock;
    const unsigned char* vals_base = reinterpret_cast<const unsigned char*>(a.vals) + (size_t)B0 * 128;
    const unsigned char* Bbytes = reinterpret_cast<const unsigned char*>(Bh);
    const size_t row_bytes = (size_t)N * 2;

    // ---- per-thread gather constants: k-row kr of both blocks, 16-byte chunk c16 of every panel ----
    const int kr = tid >> 4, c16 = tid & 15;
    const unsigned dst_off = (unsigned)((c16 >> 3) * 1024 + kr * 128 + (((c16 & 7) ^ kr) << 4));
    const unsigned idesc = (1u << 4) | (1u << 15) | (2u << 17) | (8u << 24);   // f32 acc, A MN-major, N=16, M=128

    // fetch walker: next K-step starts at block fb of unit fu (unit end fe); all threads agree
    int fu = u_lo, fb = 0, fe = 0;
    if (fu < u_hi) tc5_unit_bounds<kMode>(a, fu, B0, fb, fe);
    auto skip_empty = [&]() {
        while (fu < u_hi && fb >= fe) { ++fu; if (fu < u_hi) tc5_unit_bounds<kMode>(a, fu, B0, fb, fe); }
    };
    skip_empty();
    int nc0 = 0, nc1 = 0;                                     // gather columns of the next step
    auto load_cols = [&]() {
        if (fu < u_hi) {
            nc0 = __ldg(atox_base + (size_t)fb * kVecPerBlock + kr);
            nc1 = (fb + 1 < fe) ? __ldg(atox_base + (size_t)(fb + 1) * kVecPerBlock + kr) : -1;
        }
    };
    load_cols();
    int fstep = 0;                                            // K-steps fetched so far
    auto issue_fetch = [&]() {
        if (fu < u_hi) {
            const unsigned st = smem_s + (unsigned)((fstep % kTcStages) * stage_bytes);
            const bool has2 = fb + 1 < fe;
            for (int p = 0; p < panels; ++p) {
                const int feat = p * 128 + c16 * 8;
                if (feat < N) {
                    const unsigned d = st + (unsigned)(p * 4096) + dst_off;
                    const unsigned char* src0 = Bbytes + (size_t)nc0 * row_bytes + (size_t)feat * 2;
                    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" :: "r"(d), "l"(src0) : "memory");
                    const unsigned char* src1 = has2 ? Bbytes + (size_t)nc1 * row_bytes + (size_t)feat * 2 : Bbytes;
                    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" :: "r"(d + 2048), "l"(src1), "r"(has2 ? 16 : 0) : "memory");
                }
            }
            if (tid < 16) {
                const bool real = tid < 8 || has2;
                const unsigned char* src = real ? vals_base + (size_t)fb * 128 + tid * 16 : vals_base;
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;"
                             :: "r"(st + (unsigned)(panels * 4096) + tid * 16), "l"(src), "r"(real ? 16 : 0) : "memory");
            }
            fb += 2;
            ++fstep;
            skip_empty();
            load_cols();
        }
        cp_async_commit();
    };

#pragma unroll 1
    for (int i = 0; i < kTcStages - 1; ++i) issue_fetch();

    int cstep = 0;                                            // K-steps consumed so far
    int bad = 0;                                              // this thread saw a wait give up
    int bad_cta = 0;                                          // CTA-uniform: only ever set from a barrier reduction
    // Several units accumulate side by side in TMEM (16 columns per unit and panel) and are
    // written out together, so the wait for the tensor core and the CTA barrier that protects
    // the accumulators are paid once per batch instead of once per unit.
    const int units_per_batch = max(1, tmem_cols / (16 * panels));
    int pend_u[4], pend_steps[4];
    int slot = 0;
#pragma unroll 1
    for (int u = u_lo; u < u_hi; ++u) {
        int ub, ue;
        tc5_unit_bounds<kMode>(a, u, B0, ub, ue);
        const int nsteps = (ue - ub + 1) >> 1;
        const unsigned acc_col = (unsigned)(slot * 16 * panels);
#pragma unroll 1
        for (int s = 0; s < nsteps; ++s, ++cstep) {
            const int stage = cstep % kTcStages;
            cp_async_wait<kTcStages - 2>();
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            if (__syncthreads_or(bad)) { bad_cta = 1; break; }
            if (tid == 0) {
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const unsigned st = smem_s + (unsigned)(stage * stage_bytes);
                const unsigned long long bdesc = tc5_smem_desc(st + (unsigned)(panels * 4096), 128, 256, 0);
                for (int p = 0; p < panels; ++p) {
                    const unsigned long long adesc = tc5_smem_desc(st + (unsigned)(p * 4096), 1024, 2048, 2);
                    asm volatile("{\n\t.reg .pred q;\n\tsetp.ne.b32 q, %4, 0;\n\t"
                                 "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, q;\n\t}"
                                 :: "r"(tmem + acc_col + (unsigned)(p * 16)), "l"(adesc), "l"(bdesc), "r"(idesc),
                                    "r"(s > 0 ? 1 : 0) : "memory");
                }
                asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];"
                             :: "r"(bar0 + 8 * stage) : "memory");
            }
            // the stage of the previous step is the next to be refilled: wait for its MMAs
            if (cstep >= 1) {
                const int ps = (cstep - 1) % kTcStages;
                if (!mbar_wait(bar0 + 8 * ps, (unsigned)(((cstep - 1) / kTcStages) & 1))) bad = 1;
            }
            issue_fetch();
        }
        // Only the CTA-uniform flag leaves the loop: a thread whose own wait gave up on the last
        // K-step of a unit carries `bad` to the next barrier reduction, so every thread reaches
        // the same barriers and the aligned TMEM instructions together.
        if (bad_cta) break;
        pend_u[slot & 3] = u; pend_steps[slot & 3] = nsteps;
        ++slot;
        if (slot < units_per_batch && u + 1 < u_hi) continue;

        // ---- epilogue of the batch: TMEM -> registers -> C ----
        if (cstep > 0) {                                      // all MMAs issued so far have completed
            const int last = cstep - 1;
            if (!mbar_wait(bar0 + 8 * (last % kTcStages), (unsigned)((last / kTcStages) & 1))) bad = 1;
        }
        if (__syncthreads_or(bad)) { bad_cta = 1; break; }    // nobody reads TMEM after a failed wait
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll 1
        for (int q = 0; q < slot; ++q) {
            const int uu = pend_u[q & 3];
            float* base = a.C;
            int wrow0 = uu * kWindowRows;
            bool to_scratch = false;
            if (kMode == 2) {
                const unsigned tag = (unsigned)__ldg(a.seg_window + uu);
                wrow0 = (int)(tag & ~kSoleSegFlag) * kWindowRows;
                if (!(tag & kSoleSegFlag)) { to_scratch = true; base = a.scratch + (size_t)__ldg(a.seg_scratch + uu) * kWindowRows * N; }
            }
#pragma unroll 1
            for (int p = 0; p < panels; ++p) {
                unsigned r[8];
                if (pend_steps[q & 3] > 0) {
                    const unsigned taddr = tmem + ((unsigned)(warp * 32) << 16) + (unsigned)(q * 16 * panels + p * 16);
                    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
                                 : "r"(taddr));
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                } else {
#pragma unroll
                    for (int j = 0; j < 8; ++j) r[j] = 0u;
                }
                const int f = p * 128 + warp * 32 + lane;
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const int row = to_scratch ? j : ((kMode == 1) ? __ldg(a.win_rows + (size_t)uu * kWindowRows + j) : wrow0 + j);
                    if (!to_scratch && (row < 0 || row >= a.M)) continue;
                    if (f < N) base[(size_t)row * N + f] = __uint_as_float(r[j]);
                }
            }
        }
        slot = 0;
        // every thread has read its accumulators before the next batch overwrites them
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        __syncthreads();
    }
    cp_async_wait<0>();
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (bad_cta && tid == 0) atomicExch(status, kStatusMmaTimeout);
    if (warp == 0) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, 64;" :: "r"(tmem) : "memory");
    }
}

// ---------------------------------------------------------------------------
// Any width >= 16 and any alignment (e.g. the 47-class GCN output): one warp
// per (unit, 16-column tile), operands read straight from global memory with
// column guards, as fs_tile_spmm_kernel does (tc/ra_tc_direct.cu:109-179).
// ---------------------------------------------------------------------------
template <bool kTF32, int kMode, bool kZC>
__global__ void __launch_bounds__(128)
tile_spmm_direct_kernel(TileArgs a, const void* __restrict__ Bmat)
{
    const int u = blockIdx.x;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int N = a.N;
    const int ldb = a.ldb;                     // row stride of the B operand
    const int n0 = (blockIdx.y * 4 + warp) * 16;
    if (u >= a.num_units || n0 >= N) return;
    const int g = lane >> 2, tid = lane & 3;
    const bool p_lo = (n0 + g) < N, p_hi = (n0 + g + 8) < N;

    long long b_begin, b_end;
    int row_lo = -1, row_hi = -1;
    float* base = a.C;
    if (kMode == 2) {
        const unsigned tag = (unsigned)a.seg_window[u];
        const int w = (int)(tag & ~kSoleSegFlag);
        b_begin = a.seg_bbegin[u]; b_end = a.seg_bend[u];
        if (tag & kSoleSegFlag) {
            row_lo = w * kWindowRows + 2 * tid; row_hi = row_lo + 1;
            if (row_lo >= a.M) row_lo = -1;
            if (row_hi >= a.M) row_hi = -1;
        } else {
            base = a.scratch + (size_t)a.seg_scratch[u] * kWindowRows * N;
            row_lo = 2 * tid; row_hi = row_lo + 1;
        }
    } else {
        b_begin = a.block_offsets[u]; b_end = a.block_offsets[u + 1];
        if (kMode == 1) {
            row_lo = a.win_rows[(size_t)u * kWindowRows + 2 * tid];
            row_hi = a.win_rows[(size_t)u * kWindowRows + 2 * tid + 1];
        } else {
            row_lo = u * kWindowRows + 2 * tid; row_hi = row_lo + 1;
            if (row_lo >= a.M) row_lo = -1;
            if (row_hi >= a.M) row_hi = -1;
        }
    }

    float d[4] = {0.f, 0.f, 0.f, 0.f};
    for (long long b = b_begin; b < b_end; ++b) {
        if (!kTF32) {
            const __half* Bh = static_cast<const __half*>(Bmat);
            unsigned bfrag;
            if (kZC) {
                const unsigned long long m = __ldg(a.val_masks + b);
                const int vb0 = __ldg(a.val_base + b);
                bfrag = zc_value_bits(m, vb0, a.vals_zc, 2 * tid, g) | (zc_value_bits(m, vb0, a.vals_zc, 2 * tid + 1, g) << 16);
            } else {
                bfrag = __ldg(reinterpret_cast<const unsigned*>(a.vals + b * 64) + lane);
            }
            const int c0 = __ldg(a.atox + b * 8 + tid * 2), c1 = __ldg(a.atox + b * 8 + tid * 2 + 1);
            const __half z = __float2half(0.f);
            __half a0 = z, a1 = z, a2 = z, a3 = z;
            if (p_lo) { a0 = Bh[(size_t)c0 * ldb + n0 + g]; a1 = Bh[(size_t)c1 * ldb + n0 + g]; }
            if (p_hi) { a2 = Bh[(size_t)c0 * ldb + n0 + g + 8]; a3 = Bh[(size_t)c1 * ldb + n0 + g + 8]; }
            const unsigned f0 = ((unsigned)__half_as_ushort(a1) << 16) | __half_as_ushort(a0);
            const unsigned f1 = ((unsigned)__half_as_ushort(a3) << 16) | __half_as_ushort(a2);
            mma_f16_m16n8k8(d, f0, f1, bfrag);
        } else {
            const float* Bf = static_cast<const float*>(Bmat);
            unsigned b0, b1;
            if (kZC) {
                const unsigned long long m = __ldg(a.val_masks + b);
                const int vb0 = __ldg(a.val_base + b);
                b0 = __float_as_uint(__half2float(__ushort_as_half((unsigned short)zc_value_bits(m, vb0, a.vals_zc, tid, g))));
                b1 = __float_as_uint(__half2float(__ushort_as_half((unsigned short)zc_value_bits(m, vb0, a.vals_zc, tid + 4, g))));
            } else {
                const __half* vb = reinterpret_cast<const __half*>(a.vals + b * 64);
                const int vslot = (g * 4 + (tid >> 1)) * 2 + (tid & 1);
                b0 = __float_as_uint(__half2float(vb[vslot]));
                b1 = __float_as_uint(__half2float(vb[vslot + 4]));
            }
            const int c_lo = __ldg(a.atox + b * 8 + tid), c_hi = __ldg(a.atox + b * 8 + tid + 4);
            float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
            if (p_lo) { a0 = __ldg(Bf + (size_t)c_lo * ldb + n0 + g); a2 = __ldg(Bf + (size_t)c_hi * ldb + n0 + g); }
            if (p_hi) { a1 = __ldg(Bf + (size_t)c_lo * ldb + n0 + g + 8); a3 = __ldg(Bf + (size_t)c_hi * ldb + n0 + g + 8); }
            mma_tf32_m16n8k8(d, to_tf32_rna(a0), to_tf32_rna(a1), to_tf32_rna(a2), to_tf32_rna(a3), b0, b1);
        }
    }
    if (row_lo >= 0) {
        if (p_lo) base[(size_t)row_lo * N + n0 + g] = d[0];
        if (p_hi) base[(size_t)row_lo * N + n0 + g + 8] = d[2];
    }
    if (row_hi >= 0) {
        if (p_lo) base[(size_t)row_hi * N + n0 + g] = d[1];
        if (p_hi) base[(size_t)row_hi * N + n0 + g + 8] = d[3];
    }
}

// Deterministic merge of split-window partial tiles (replaces
// sh_merge_split_kernel, tc/ra_segment_hybrid.cu:198-221): slots summed in
// ascending order.
__global__ void __launch_bounds__(256)
tile_merge_kernel(const int* __restrict__ split_wins, const int* __restrict__ split_off,
                  const float* __restrict__ scratch, float* __restrict__ C,
                  int num_split, int M, int N)
{
    const long long total = (long long)num_split * kWindowRows * N;
    for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
         idx += (long long)gridDim.x * blockDim.x) {
        const int sw = (int)(idx / ((long long)kWindowRows * N));
        const long long rem = idx - (long long)sw * kWindowRows * N;
        const int slot = (int)(rem / N);
        const int col = (int)(rem - (long long)slot * N);
        const int r = split_wins[sw] * kWindowRows + slot;
        if (r >= M) continue;
        float acc = 0.f;
        const int o_end = split_off[sw + 1];
        for (int o = split_off[sw]; o < o_end; ++o) {
            acc += scratch[((long long)o * kWindowRows + slot) * N + col];
        }
        C[(long long)r * N + col] = acc;
    }
}

// Same merge for N % 4 == 0 and 16-byte aligned C / scratch: one thread sums a float4 column
// group, four partial tiles in flight at a time (the partials of a hub window are 8 x N floats
// 8*N floats apart, so the loads of one thread are independent); the additions stay in
// ascending slot order, as in the scalar kernel.
__global__ void __launch_bounds__(256)
tile_merge_vec4_kernel(const int* __restrict__ split_wins, const int* __restrict__ split_off,
                       const float4* __restrict__ scratch, float4* __restrict__ C,
                       int num_split, int M, int N4)
{
    const long long total = (long long)num_split * kWindowRows * N4;
    for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
         idx += (long long)gridDim.x * blockDim.x) {
        const int sw = (int)(idx / ((long long)kWindowRows * N4));
        const long long rem = idx - (long long)sw * kWindowRows * N4;
        const int slot = (int)(rem / N4);
        const int col = (int)(rem - (long long)slot * N4);
        const int r = __ldg(split_wins + sw) * kWindowRows + slot;
        if (r >= M) continue;
        const int o_begin = __ldg(split_off + sw), o_end = __ldg(split_off + sw + 1);
        const long long stride = (long long)kWindowRows * N4;
        const float4* src = scratch + ((long long)o_begin * kWindowRows + slot) * N4 + col;
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        int o = o_begin;
        for (; o + 4 <= o_end; o += 4, src += 4 * stride) {
            const float4 p0 = __ldcs(src), p1 = __ldcs(src + stride), p2 = __ldcs(src + 2 * stride), p3 = __ldcs(src + 3 * stride);
            acc.x += p0.x; acc.y += p0.y; acc.z += p0.z; acc.w += p0.w;
            acc.x += p1.x; acc.y += p1.y; acc.z += p1.z; acc.w += p1.w;
            acc.x += p2.x; acc.y += p2.y; acc.z += p2.z; acc.w += p2.w;
            acc.x += p3.x; acc.y += p3.y; acc.z += p3.z; acc.w += p3.w;
        }
        for (; o < o_end; ++o, src += stride) {
            const float4 p = __ldcs(src);
            acc.x += p.x; acc.y += p.y; acc.z += p.z; acc.w += p.w;
        }
        C[(long long)r * N4 + col] = acc;
    }
}

// B fp32 -> fp16, round to nearest even (replaces convert_b_to_half_kernel,
// tc/ra_tc_direct.cu:85-104): 8 elements per thread, 2x128-bit in, 128-bit out.
__global__ void __launch_bounds__(256)
convert_b_to_half_kernel(const float* __restrict__ B, __half* __restrict__ Bh, long long total, int vec_ok)
{
    const long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const long long nthreads = (long long)gridDim.x * blockDim.x;
    long long done = 0;
    if (vec_ok) {
        const long long groups = total / 8;
        for (long long gi = tid; gi < groups; gi += nthreads) {
            const float4 x = __ldcs(reinterpret_cast<const float4*>(B) + 2 * gi);
            const float4 y = __ldcs(reinterpret_cast<const float4*>(B) + 2 * gi + 1);
            __half2 h0 = __floats2half2_rn(x.x, x.y), h1 = __floats2half2_rn(x.z, x.w);
            __half2 h2 = __floats2half2_rn(y.x, y.y), h3 = __floats2half2_rn(y.z, y.w);
            uint4 o;
            o.x = *reinterpret_cast<unsigned*>(&h0); o.y = *reinterpret_cast<unsigned*>(&h1);
            o.z = *reinterpret_cast<unsigned*>(&h2); o.w = *reinterpret_cast<unsigned*>(&h3);
            reinterpret_cast<uint4*>(Bh)[gi] = o;
        }
        done = groups * 8;
    }
    for (long long i = done + tid; i < total; i += nthreads) Bh[i] = __float2half_rn(B[i]);
}

// B fp32 [K,N] -> fp16 [K,ldb] with zero-filled pad columns (ldb = N rounded up to 16): gives
// the staged kernel 16-byte aligned rows for widths such as the 47-class GCN output.
__global__ void __launch_bounds__(256)
convert_b_to_half_padded_kernel(const float* __restrict__ B, __half* __restrict__ Bh, long long K, int N, int ldb)
{
    const long long total = K * ldb;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (long long)gridDim.x * blockDim.x) {
        const long long r = i / ldb;
        const int c = (int)(i - r * ldb);
        Bh[i] = (c < N) ? __float2half_rn(__ldcs(B + r * N + c)) : __float2half(0.f);
    }
}

template <bool kTF32, int kMode, bool kZC = false>
static int launch_tile(const TileArgs& a, const void* B, bool staged, cudaStream_t st, int* status)
{
    if (staged) {
        constexpr int elem = kTF32 ? 4 : 2;
        constexpr int stage = kTF32 ? kStageF32 : kStageF16;
        const int slices = (a.ldb * elem + 127) / 128;
        RA_REQUIRE(slices <= 8, RA_ERR_UNSUPPORTED, "tile SpMM: N=%d too wide for the staged kernel", a.N);
        const bool padded = a.ldb != a.N;                    // only the per-warp ring takes a padded operand
        const int groups_per_cta = std::max(1, 4 / slices);
        const int warps = slices * groups_per_cta;
        // TF32: 4 stages at N = 256 (8 slices) and on SEGMENT_HYBRID, else 8; FP16: 8
        const int depth = (kTF32 && (slices >= 8 || kMode == 2)) ? 4 : 8;
        const size_t smem = (size_t)warps * depth * stage;
        const long long weight = a.total_blocks + a.num_units;
        const int ctas_per_sm = (int)std::max<size_t>(1, std::min<size_t>(8, (200 * 1024) / smem));
        long long groups = (long long)sm_count() * ctas_per_sm * groups_per_cta * 3;
        groups = std::min(groups, std::max<long long>(1, weight / 48));
        const int ctas = (int)((groups + groups_per_cta - 1) / groups_per_cta);
        groups = (long long)ctas * groups_per_cta;
        // Engine choice, from full-size measurements on B200 (ms, TMA gather ring / cp.async ring / tcgen05):
        //   FP16  N=256: configuration 3 COMMUNITY_TC 5.0 / 6.4 / -, configuration 5 10.2 / 13.4 / -
        //         N=128: configuration 3 4.0 / 3.9 / 5.7, configuration 5 6.1 / 7.0 / 7.4, configuration 2 0.69 / 1.72 / 1.16
        //         N=64 : configuration 4 TC_DIRECT 4.9 / 11.4 / -
        //   TF32  N=64 : configuration 4 SEGMENT_HYBRID 4.7 / 5.0, configuration 3 4.3 / 4.6
        //         N=128: configuration 3 8.5 / 9.2, configuration 2 0.93 / 1.13 (SEGMENT_HYBRID on 4: 9.2 / 8.9)
        //         N=256: configuration 3 17.3 / 15.9, configuration 4 19.9 / 19.0
        //   a few thousand blocks (configuration 1): 0.039 / 0.026
        // So: the TMA ring for FP16 and for TF32 rows up to 512 bytes, the cp.async ring for wider TF32
        // rows, for small matrices and for rows that are not whole 128-byte slices (N=47: 4.9 vs 3.6).
        // The tcgen05 / TMEM kernel (FP16, N <= 512) was ahead of the rings at N=128 before they got
        // their deeper stages and index batches; it is kept behind RA_TILE_TC5=1.
        // RA_TILE_G4=1/0 forces the TMA ring on or off.
        const char* tc5_env = std::getenv("RA_TILE_TC5");
        const bool use_tc5 = !kZC && !padded && !kTF32 && a.N <= 512 && tc5_env && tc5_env[0] == '1';
        const char* g4_env = std::getenv("RA_TILE_G4");
        // The TMA ring shares windows between groups (partial tiles in scratch, merged in block order),
        // so hub windows of thousands of blocks are no obstacle. Without room for the partial tiles
        // (RA_G4_SPLIT=0) a warp walks a long window alone with three blocks in flight, and the cp.async
        // ring keeps those shapes.
        const bool shares_windows = kMode != 2 && a.scratch != nullptr && a.scratch_floats > 0;
        const bool whole_units_ok = kMode == 2 || shares_windows || a.max_unit_blocks <= 1024;
        const long long min_weight = std::getenv("RA_G4_MIN_WEIGHT") ? std::atoll(std::getenv("RA_G4_MIN_WEIGHT")) : 16384ll;
        const bool g4_auto = !use_tc5 && whole_units_ok && a.total_blocks + a.num_units >= min_weight &&
                             (!kTF32 || a.N <= 128) && (a.ldb * elem) % 128 == 0;
        const bool use_g4 = !kZC && (g4_env ? (g4_env[0] == '1') : g4_auto);
        if (use_g4) {
            const int rc = launch_tile_gather4<kTF32, kMode>(a, B, a.K, st, status);
            if (rc != RA_ERR_UNSUPPORTED) return rc;
        }
        if (use_tc5) {
            const int panels = (a.N + 127) / 128;
            const size_t smem5 = (size_t)kTcStages * (panels * 4096 + 1024) + 1024;
            const int per_sm = (int)std::max<size_t>(1, std::min<size_t>(8, (200 * 1024) / (smem5 + 1024)));
            long long ctas5 = (long long)sm_count() * per_sm * 3;
            ctas5 = std::min(ctas5, std::max<long long>(1, weight / 48));
            auto kern5 = tile_spmm_tc5_kernel<kMode>;
            static std::atomic<unsigned long long> attr_set5{0};
            RA_CUDA_TRY(configure_once_per_device(attr_set5, [&]() {
                return cudaFuncSetAttribute(kern5, cudaFuncAttributeMaxDynamicSharedMemorySize, 100 * 1024);
            }));
            kern5<<<(unsigned)ctas5, kTcThreads, smem5, st>>>(a, static_cast<const __half*>(B), (int)ctas5, panels, status);
            RA_KERNEL_CHECK();
            return RA_OK;
        }
        // The bulk-copy (TMA) ring is kept as a measured alternative: on B200 it is 20-55 % slower than
        // the per-warp cp.async ring at the same bytes in flight, so it is off unless RA_TILE_TMA=1.
        const char* tma_env = std::getenv("RA_TILE_TMA");
        const bool use_tma = tma_env && tma_env[0] == '1';
        if (!kZC && !padded && use_tma) {
            const int pad = kTF32 ? 32 : 16;
            const int stage_bytes = 8 * (a.N * elem + pad) + 128;
            const int group_bytes = ((128 + kStages * stage_bytes) + 127) & ~127;
            const size_t smem_t = (size_t)groups_per_cta * group_bytes;
            const int ctas_per_sm_t = (int)std::max<size_t>(1, std::min<size_t>(8, (200 * 1024) / smem_t));
            long long groups_t = (long long)sm_count() * ctas_per_sm_t * groups_per_cta * 3;
            groups_t = std::min(groups_t, std::max<long long>(1, weight / 48));
            const int ctas_t = (int)((groups_t + groups_per_cta - 1) / groups_per_cta);
            groups_t = (long long)ctas_t * groups_per_cta;
            auto kern_t = tile_spmm_tma_kernel<kTF32, kMode>;
            static std::atomic<unsigned long long> attr_set_t{0};
            RA_CUDA_TRY(configure_once_per_device(attr_set_t, [&]() {
                return cudaFuncSetAttribute(kern_t, cudaFuncAttributeMaxDynamicSharedMemorySize, 100 * 1024);
            }));
            RA_REQUIRE(smem_t <= 100 * 1024, RA_ERR_UNSUPPORTED, "tile SpMM: N=%d too wide for the staged kernel", a.N);
            // RA_TILE_TMA_POLL_LIMIT (tests only): polls a consumer warp spends on a stage before it
            // gives up and reports through the status word (0 = gives up at once); every other
            // wait keeps the normal limit
            const char* poll_env = std::getenv("RA_TILE_TMA_POLL_LIMIT");
            const int poll_limit = poll_env ? std::max(0, std::atoi(poll_env)) : kSpinLimit;
            kern_t<<<ctas_t, warps * 32, smem_t, st>>>(a, B, slices, (int)groups_t, group_bytes, status, poll_limit);
            RA_KERNEL_CHECK();
            return RA_OK;
        }
        if (kTF32 && depth == 4) {
            auto kern = tile_spmm_kernel<kTF32, kMode, kZC, kTF32 ? 4 : 8>;
            static std::atomic<unsigned long long> attr_set4{0};
            RA_CUDA_TRY(configure_once_per_device(attr_set4, [&]() {
                return cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 8 * 4 * stage);
            }));
            kern<<<ctas, warps * 32, smem, st>>>(a, B, slices, (int)groups);
        } else {
            auto kern = tile_spmm_kernel<kTF32, kMode, kZC, 8>;
            static std::atomic<unsigned long long> attr_set{0};
            RA_CUDA_TRY(configure_once_per_device(attr_set, [&]() {
                return cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 8 * 8 * stage);
            }));
            kern<<<ctas, warps * 32, smem, st>>>(a, B, slices, (int)groups);
        }
    } else {
        dim3 grid((unsigned)a.num_units, (unsigned)((a.N + 63) / 64));
        tile_spmm_direct_kernel<kTF32, kMode, kZC><<<grid, 128, 0, st>>>(a, B);
    }
    RA_KERNEL_CHECK();
    return RA_OK;
}

}  // namespace ra

extern "C" int ra_tile_plan_run(RaTilePlan* p, int precision, const void* d_B, int b_dtype,
                                float* d_C, int N, void* stream)
{
    using namespace ra;
    RA_REQUIRE(p != nullptr, RA_ERR_INVALID_ARG, "ra_tile_plan_run: plan is null");
    RA_REQUIRE(precision == RA_PRECISION_FP16 || precision == RA_PRECISION_TF32, RA_ERR_INVALID_ARG,
               "ra_tile_plan_run: unknown precision %d", precision);
    RA_REQUIRE(b_dtype == RA_DTYPE_F32 || (b_dtype == RA_DTYPE_F16 && precision == RA_PRECISION_FP16),
               RA_ERR_INVALID_ARG, "ra_tile_plan_run: fp16 B is accepted on the FP16 path only");
    RA_REQUIRE(p->active, RA_ERR_INACTIVE_PLAN,
               "ra_tile_plan_run: the plan is inactive (built with N < 16 or an empty matrix)");
    RA_REQUIRE(N >= 16, RA_ERR_UNSUPPORTED, "ra_tile_plan_run: N=%d is below the tile minimum of 16", N);
    RA_REQUIRE(d_B && d_C, RA_ERR_INVALID_ARG, "ra_tile_plan_run: null pointer");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const bool tf32 = precision == RA_PRECISION_TF32;

    const void* Bop = d_B;
    // widths that are not a multiple of 16 get a padded fp16 copy of B (the conversion pass runs
    // anyway), so they run on the staged kernel instead of the direct-load fallback. Where rounding
    // the row up to whole 128-byte slices costs at most 40 % more bytes (N=47 -> 64, N=100 -> 128) the
    // copy is padded that far and the TMA ring takes it: configuration 5, 3.1 vs 3.6 ms and 5.3 vs 7.5 ms.
    int ldb = N;
    if (!tf32 && b_dtype == RA_DTYPE_F32) {
        ldb = (N + 15) & ~15;
        const int slices = (N + 63) & ~63;
        if (ldb % 64 != 0 && N > 32 && (long long)slices * 5 <= (long long)N * 7 && !(std::getenv("RA_TILE_PAD_SLICES") && std::getenv("RA_TILE_PAD_SLICES")[0] == '0')) ldb = slices;
    }
    if (!tf32 && b_dtype == RA_DTYPE_F32) {
        const long long total = (long long)p->K * ldb;
        const size_t need = (size_t)total * sizeof(uint16_t);
        if (need > p->bhalf_bytes) {
            if (p->d_bhalf) RA_CUDA_TRY(cudaFree(p->d_bhalf));
            p->d_bhalf = nullptr; p->bhalf_bytes = 0;
            RA_CUDA_TRY(cudaMalloc(reinterpret_cast<void**>(&p->d_bhalf), need));
            p->bhalf_bytes = need;
        }
        const long long groups = (total + 7) / 8;
        const int blocks = (int)std::min<long long>((groups + 255) / 256, (long long)sm_count() * 16);
        if (ldb != N) {
            const int pblocks = (int)std::min<long long>((total + 255) / 256, (long long)sm_count() * 32);
            convert_b_to_half_padded_kernel<<<std::max(pblocks, 1), 256, 0, st>>>(
                static_cast<const float*>(d_B), reinterpret_cast<__half*>(p->d_bhalf), p->K, N, ldb);
        } else {
            convert_b_to_half_kernel<<<std::max(blocks, 1), 256, 0, st>>>(
                static_cast<const float*>(d_B), reinterpret_cast<__half*>(p->d_bhalf), total,
                (aligned16(d_B) && aligned16(p->d_bhalf)) ? 1 : 0);
        }
        RA_KERNEL_CHECK();
        Bop = p->d_bhalf;
    }
    if (p->kind == RA_TILE_SEGMENT_HYBRID && p->num_split_segs > 0) {
        const size_t need = (size_t)p->num_split_segs * kWindowRows * (size_t)N * sizeof(float);
        if (need > p->scratch_bytes) {
            if (p->d_scratch) RA_CUDA_TRY(cudaFree(p->d_scratch));
            p->d_scratch = nullptr; p->scratch_bytes = 0;
            RA_CUDA_TRY(cudaMalloc(reinterpret_cast<void**>(&p->d_scratch), need));
            p->scratch_bytes = need;
        }
    }

    TileArgs a{};
    a.block_offsets = p->d_block_offsets; a.atox = p->d_atox; a.vals = p->d_vals_f16;
    a.val_masks = p->d_val_masks; a.val_base = p->d_val_base; a.vals_zc = p->d_vals_zc;
    a.win_rows = p->d_win_rows;
    a.seg_window = p->d_seg_window; a.seg_bbegin = p->d_seg_bbegin; a.seg_bend = p->d_seg_bend;
    a.seg_scratch = p->d_seg_scratch;
    a.num_units = (p->kind == RA_TILE_SEGMENT_HYBRID) ? p->num_segments : p->num_windows;
    a.M = p->M; a.K = p->K; a.N = N; a.ldb = ldb; a.total_blocks = p->num_blocks;
    a.max_unit_blocks = (p->kind == RA_TILE_SEGMENT_HYBRID) ? std::min(p->max_window_blocks, kSegBlocks) : p->max_window_blocks;
    if (p->kind == RA_TILE_TC_DIRECT || p->kind == RA_TILE_COMMUNITY_TC) {
        // room for the partial tiles of windows that the TMA ring shares between groups
        const size_t need = (size_t)tile_gather4_split_scratch_floats(tf32, p->kind == RA_TILE_COMMUNITY_TC ? 1 : 0, a) * sizeof(float);
        if (need > p->scratch_bytes) {
            if (p->d_scratch) RA_CUDA_TRY(cudaFree(p->d_scratch));
            p->d_scratch = nullptr; p->scratch_bytes = 0;
            RA_CUDA_TRY(cudaMalloc(reinterpret_cast<void**>(&p->d_scratch), need));
            p->scratch_bytes = need;
        }
    }
    a.C = d_C; a.scratch = p->d_scratch; a.scratch_floats = (long long)(p->scratch_bytes / sizeof(float));

    // RA_TC_STAGED=0 keeps the direct-load kernels, as in the reference (tc/ra_tc_direct.cu:837-838)
    const char* staged_env = std::getenv("RA_TC_STAGED");
    const bool staged_off = staged_env && staged_env[0] == '0';
    const bool staged = !staged_off && (ldb % 16 == 0) && aligned16(Bop) && (ldb * (tf32 ? 4 : 2) <= 1024) &&
                        (!tf32 || aligned16(d_C));            // the TF32 kernel stores 128-bit row pieces
    int rc;
    if (p->kind == RA_TILE_TC_DIRECT_ZC)
        rc = tf32 ? launch_tile<true, 0, true>(a, Bop, staged, st, p->d_status) : launch_tile<false, 0, true>(a, Bop, staged, st, p->d_status);
    else if (p->kind == RA_TILE_TC_DIRECT)
        rc = tf32 ? launch_tile<true, 0>(a, Bop, staged, st, p->d_status) : launch_tile<false, 0>(a, Bop, staged, st, p->d_status);
    else if (p->kind == RA_TILE_COMMUNITY_TC)
        rc = tf32 ? launch_tile<true, 1>(a, Bop, staged, st, p->d_status) : launch_tile<false, 1>(a, Bop, staged, st, p->d_status);
    else
        rc = tf32 ? launch_tile<true, 2>(a, Bop, staged, st, p->d_status) : launch_tile<false, 2>(a, Bop, staged, st, p->d_status);
    if (rc != RA_OK) return rc;

    if (p->kind == RA_TILE_SEGMENT_HYBRID && p->num_split_windows > 0) {
        if (N % 4 == 0 && aligned16(d_C) && aligned16(p->d_scratch)) {
            const long long total = (long long)p->num_split_windows * kWindowRows * (N / 4);
            const int blocks = (int)std::min<long long>((total + 255) / 256, (long long)sm_count() * 16);
            tile_merge_vec4_kernel<<<std::max(blocks, 1), 256, 0, st>>>(
                p->d_split_wins, p->d_split_off, reinterpret_cast<const float4*>(p->d_scratch),
                reinterpret_cast<float4*>(d_C), p->num_split_windows, p->M, N / 4);
        } else {
            const long long total = (long long)p->num_split_windows * kWindowRows * N;
            const int blocks = (int)std::min<long long>((total + 255) / 256, (long long)sm_count() * 16);
            tile_merge_kernel<<<std::max(blocks, 1), 256, 0, st>>>(p->d_split_wins, p->d_split_off, p->d_scratch,
                                                                   d_C, p->num_split_windows, p->M, N);
        }
        RA_KERNEL_CHECK();
    }
    return RA_OK;
}
