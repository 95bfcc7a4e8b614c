// Streaming row engine with shared-memory staging of the gathered B rows.
//
// A warp takes a batch of up to 32 "segments" (rows of A, or <=256-nnz chunks
// of long rows) and treats their nonzeros as one stream. Every nonzero needs
// one dense row of B (N floats): the warp copies those rows into a private
// shared-memory ring (16 rows) with 16-byte cp.async (one 512-byte row per warp
// instruction at N=128) and keeps the ring full: 12 rows are always in flight
// while the oldest group of 4 is being multiplied, so the number of bytes in
// flight per SM no longer depends on registers or on how short the rows are.
// At segment boundaries the accumulators are flushed to the segment's
// destination (a row of C, or a scratch slot for a chunk of a multi-chunk row).
//
// Stream coordinates
//   kContig (CSR_DIRECT, consecutive rows): the coordinate is the nonzero
//     index itself; a lane loads 4 consecutive (col, val) pairs with one
//     aligned 128-bit streaming load each, 128 nonzeros per warp step;
//   otherwise (listed rows, chunks): the coordinate is the running sum of the
//     segment lengths; every lane loads its 4 pairs from its segment.
// In both cases an element finds its segment by a 5-step search over the
// segment start coordinates that the lanes hold (warp shuffles).
//
// Replaces the gather loops of csr_direct_subwarp_vec4_kernel
// (csr/csr_direct.cu:201-224), zo_small_subwarp_vec4_kernel and
// zo_chunk_vec4_kernel (csr/ra_zero_overhead.cu:93-150, 226-268) for
// N in {128, 256, 512}.
#pragma once

#include "common.cuh"

#include <algorithm>

namespace ra {

constexpr int kStreamWarps   = 4;                 // warps per CTA
constexpr int kStreamThreads = kStreamWarps * 32;
constexpr int kStreamSlots   = 16;                // ring slots (one B row each) per warp
constexpr int kStreamGroups  = kStreamSlots / 4;  // groups of 4 slots
constexpr int kStreamSetBytes = 128 * 8;          // (value, segment) of one 128-element step
constexpr unsigned kStreamSoleFlag = 0x80000000u;
constexpr int kStreamChunk   = 256;

// kModeFused: one launch whose first chunk_warps warps take the chunks and whose other
// warps take the listed rows (the two data phases of a ZERO_OVERHEAD_CSR run).
enum StreamMode { kModeRows = 0, kModeListed = 1, kModeChunks = 2, kModeFused = 3 };

inline int stream_warp_smem(int V) { return kStreamSlots * 512 * V + kStreamSetBytes; }

struct StreamArgs {
    const int* rowptr;
    const int* colind;
    const float* vals;
    const float* B;
    float* C;
    float* scratch;            // chunks of multi-chunk rows
    const int* row_ids;        // kModeListed (nullptr = consecutive rows)
    const int* chunk_rows;     // kModeChunks
    const int* chunk_starts;
    const int* chunk_slot;
    long long num_items;       // rows or chunks
    int N;
    int segs_per_batch;        // <= 32
    int batches_per_warp;
    long long weight_per_warp; // kModeRows: rows are dealt to warps by (nonzeros + rows); 0 = by count
    long long num_chunks;      // kModeFused: chunks (num_items = listed rows)
    long long chunk_warps;     // kModeFused: warps [0, chunk_warps) take chunks
    int chunk_batches_per_warp;
};

struct ASet {                  // 4 stream elements per lane
    int c[4];                  // column, -1 = no element
    float v[4];
    int seg[4];                // segment index inside the batch, -1 = no element
};

__device__ __forceinline__ void stream_cp_async_16(unsigned smem_addr, const void* g) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" :: "r"(smem_addr), "l"(g) : "memory");
}
__device__ __forceinline__ void stream_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int kPending>
__device__ __forceinline__ void stream_wait() { asm volatile("cp.async.wait_group %0;" :: "n"(kPending) : "memory"); }

// V = float4 per lane (N = 128*V); kMode as above.
template <int V, int kMode>
__global__ void __launch_bounds__(kStreamThreads, (V == 1) ? 6 : ((V == 2) ? 3 : 1))
csr_stream_kernel(StreamArgs a)
{
    constexpr int R  = kStreamSlots;
    constexpr int NG = kStreamGroups;
    constexpr int kRowBytes = 512 * V;
    constexpr int kWarpSmem = R * kRowBytes + kStreamSetBytes;
    constexpr bool kContig = (kMode == kModeRows);
    extern __shared__ __align__(16) unsigned char smem[];

    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    unsigned char* ring_ptr = smem + warp * kWarpSmem;
    const unsigned ring = (unsigned)__cvta_generic_to_shared(ring_ptr);
    float2* set_sm = reinterpret_cast<float2*>(ring_ptr + R * kRowBytes);   // [128] (value, segment)
    const long long gwarp = (long long)blockIdx.x * kStreamWarps + warp;
    const int N = a.N;
    const int spb = a.segs_per_batch;
    const unsigned char* Bbytes = reinterpret_cast<const unsigned char*>(a.B);
    const size_t b_row_bytes = (size_t)N * 4;

    // segment metadata of one batch: lane j owns segment j
    auto load_meta = [&](long long first, long long limit, int& s, int& e, float*& dst) {
        s = 0; e = 0; dst = nullptr;
        const long long it = first + lane;
        if (lane < spb && it < limit) {
            if (kMode == kModeChunks) {
                const unsigned tag = (unsigned)__ldg(a.chunk_rows + it);
                const int row = (int)(tag & ~kStreamSoleFlag);
                s = __ldg(a.chunk_starts + it);
                e = min(s + kStreamChunk, __ldg(a.rowptr + row + 1));
                const int slot = __ldg(a.chunk_slot + it);
                dst = (slot < 0) ? a.C + (size_t)row * N : a.scratch + (size_t)slot * N;
            } else {
                const int row = (kMode == kModeListed && a.row_ids) ? __ldg(a.row_ids + it) : (int)it;
                s = __ldg(a.rowptr + row);
                e = __ldg(a.rowptr + row + 1);
                dst = a.C + (size_t)row * N;
            }
        }
    };

    // this warp's item range
    long long it_lo, it_hi;
    if (kMode == kModeRows && a.weight_per_warp > 0) {
        // rows are dealt out by weight = nonzeros + rows, so hub rows do not pile
        // up in one warp; a row is never split
        const int base = __ldg(a.rowptr);
        auto weight_lower_bound = [&](long long target) -> long long {
            long long lo = 0, hi = a.num_items;     // smallest r with rowptr[r]-rowptr[0]+r >= target
            while (lo < hi) {
                const long long mid = (lo + hi) >> 1;
                if ((long long)(__ldg(a.rowptr + mid) - base) + mid < target) lo = mid + 1; else hi = mid;
            }
            return lo;
        };
        it_lo = weight_lower_bound(gwarp * a.weight_per_warp);
        it_hi = weight_lower_bound((gwarp + 1) * a.weight_per_warp);
        // the last warp of the grid closes the range whatever nnz the caller stated
        if (gwarp == (long long)gridDim.x * kStreamWarps - 1) it_hi = a.num_items;
    } else {
        it_lo = gwarp * a.batches_per_warp * spb;
        it_hi = min(a.num_items, it_lo + (long long)a.batches_per_warp * spb);
    }
    if (it_lo >= it_hi) return;
    int s_n, e_n; float* dst_n;
    load_meta(it_lo, it_hi, s_n, e_n, dst_n);

#pragma unroll 1
    for (long long first = it_lo; first < it_hi; first += spb) {
        const int count = (int)min((long long)spb, it_hi - first);
        const int s = s_n, e = e_n;
        float* dst = dst_n;
        if (first + spb < it_hi) load_meta(first + spb, it_hi, s_n, e_n, dst_n);   // prefetch

        const int len = e - s;
        int seg_begin;                     // segment start in stream coordinates
        int x0, x_end;                     // stream range [x0, x_end)
        int first_valid;                   // elements below this coordinate are padding
        if (kContig) {
            seg_begin = (lane < count) ? s : 0x7fffffff;
            const int s0 = __shfl_sync(0xffffffffu, s, 0);
            x_end = __shfl_sync(0xffffffffu, e, count - 1);
            x0 = s0 & ~3;
            first_valid = s0;
        } else {
            int inc = len;
#pragma unroll
            for (int off = 1; off < 32; off <<= 1) {
                const int y = __shfl_up_sync(0xffffffffu, inc, off);
                if (lane >= off) inc += y;
            }
            seg_begin = (lane < count) ? (inc - len) : 0x7fffffff;
            x0 = 0;
            first_valid = 0;
            x_end = __shfl_sync(0xffffffffu, inc, 31);
        }
        const int total = x_end - x0;                       // stream length incl. head padding
        const int num_groups = (total + 3) >> 2;

        auto find_seg = [&](int x) -> int {                 // last j < count with seg_begin[j] <= x
            int lo = 0;
#pragma unroll
            for (int st = 16; st > 0; st >>= 1) {
                const int cand = lo + st;
                const int bv = __shfl_sync(0xffffffffu, seg_begin, cand & 31);
                if (cand < count && bv <= x) lo = cand;
            }
            return lo;
        };
        auto load_set = [&](int step) -> ASet {
            ASet st;
            const int xb = x0 + step * 128 + 4 * lane;      // first coordinate of this lane
            int4 c4 = make_int4(0, 0, 0, 0);
            int4 v4 = make_int4(0, 0, 0, 0);
            if (kContig) {
                if (xb < x_end) {
                    c4 = __ldcs(reinterpret_cast<const int4*>(a.colind + xb));
                    v4 = __ldcs(reinterpret_cast<const int4*>(a.vals + xb));
                }
            }
            const int cc[4] = {c4.x, c4.y, c4.z, c4.w};
            const int vv[4] = {v4.x, v4.y, v4.z, v4.w};
            // consecutive coordinates mostly share a segment: search once per lane,
            // then only re-search when the next coordinate leaves the segment
            int j = find_seg(xb);
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const int x = xb + k;
                if (k > 0) j = find_seg(x);                 // all lanes take part in the shuffles
                const bool ok = (x >= first_valid) && (x < x_end);
                st.seg[k] = ok ? j : -1;
                if (kContig) {
                    st.c[k] = ok ? cc[k] : -1;
                    st.v[k] = __int_as_float(vv[k]);
                } else {
                    const int sj = __shfl_sync(0xffffffffu, s, j);
                    const int bj = __shfl_sync(0xffffffffu, seg_begin, j);
                    st.c[k] = -1; st.v[k] = 0.f;
                    if (ok) {
                        const int p = sj + (x - bj);
                        st.c[k] = __ldcs(a.colind + p);
                        st.v[k] = __ldcs(a.vals + p);
                    }
                }
            }
            return st;
        };
        // (value, segment) of the step being consumed live in shared memory so the
        // consumer reads them with broadcast loads instead of shuffles
        auto publish_set = [&](const ASet& st) {
            float4* out = reinterpret_cast<float4*>(set_sm + 4 * lane);
            out[0] = make_float4(st.v[0], __int_as_float(st.seg[0]), st.v[1], __int_as_float(st.seg[1]));
            out[1] = make_float4(st.v[2], __int_as_float(st.seg[2]), st.v[3], __int_as_float(st.seg[3]));
        };

        ASet cur = load_set(0);
        ASet nxt;
        if (total > 128) nxt = load_set(1);
        else {
#pragma unroll
            for (int k = 0; k < 4; ++k) { nxt.c[k] = -1; nxt.v[k] = 0.f; nxt.seg[k] = -1; }
        }
        __syncwarp();
        publish_set(cur);
        __syncwarp();

        auto fetch = [&](int gf, int consume_step) {
            const bool use_cur = (gf >> 5) == consume_step;
            const int src = gf & 31;
            const unsigned slot0 = ring + (unsigned)(((gf * 4) % R) * kRowBytes) + lane * 16;
            int cols[4];
            if (use_cur) {                                  // warp-uniform
#pragma unroll
                for (int k = 0; k < 4; ++k) cols[k] = __shfl_sync(0xffffffffu, cur.c[k], src);
            } else {
#pragma unroll
                for (int k = 0; k < 4; ++k) cols[k] = __shfl_sync(0xffffffffu, nxt.c[k], src);
            }
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const int col = cols[k];
                if (col >= 0) {
                    const unsigned char* g = Bbytes + (size_t)col * b_row_bytes + lane * 16;
#pragma unroll
                    for (int v = 0; v < V; ++v) stream_cp_async_16(slot0 + k * kRowBytes + v * 512, g + v * 512);
                }
            }
        };

#pragma unroll 1
        for (int gf = 0; gf < NG; ++gf) {
            if (gf < num_groups) fetch(gf, 0);
            stream_commit();
        }

        float4 acc[V];
#pragma unroll
        for (int v = 0; v < V; ++v) acc[v] = make_float4(0.f, 0.f, 0.f, 0.f);
        int cur_seg = -1;
        auto flush = [&](int seg) {
            const unsigned long long d =
                ((unsigned long long)__shfl_sync(0xffffffffu, (unsigned)((unsigned long long)dst >> 32), seg) << 32) |
                (unsigned long long)__shfl_sync(0xffffffffu, (unsigned)((unsigned long long)dst & 0xffffffffu), seg);
            float4* out = reinterpret_cast<float4*>(d) + lane;
#pragma unroll
            for (int v = 0; v < V; ++v) st_stream_float4(out + v * 32, acc[v]);
        };

        // one round = the NG groups of the ring, so slot addresses are static
#pragma unroll 1
        for (int g0 = 0; g0 < num_groups; g0 += NG) {
            if (g0 > 0 && (g0 & 31) == 0) {
                cur = nxt;
                __syncwarp();
                publish_set(cur);
                const int step = (g0 >> 5) + 1;
                if (step * 128 < total) nxt = load_set(step);
            }
            const int cstep = g0 >> 5;
            const float2* set_round = set_sm + (g0 & 31) * 4;
#pragma unroll
            for (int j = 0; j < NG; ++j) {
                const int gc = g0 + j;
                if (gc < num_groups) {                           // warp-uniform
                    stream_wait<NG - 1>();
                    __syncwarp();
                    const unsigned char* slot0 = ring_ptr + (j * 4) * kRowBytes + lane * 16;
                    const float4 p01 = *reinterpret_cast<const float4*>(set_round + j * 4);
                    const float4 p23 = *reinterpret_cast<const float4*>(set_round + j * 4 + 2);
                    float4 b[4][V];
#pragma unroll
                    for (int k = 0; k < 4; ++k)
#pragma unroll
                        for (int v = 0; v < V; ++v)
                            b[k][v] = *reinterpret_cast<const float4*>(slot0 + k * kRowBytes + v * 512);
                    const float av[4] = {p01.x, p01.z, p23.x, p23.z};
                    const int sg[4] = {__float_as_int(p01.y), __float_as_int(p01.w),
                                       __float_as_int(p23.y), __float_as_int(p23.w)};
                    if (cur_seg >= 0 && sg[0] == cur_seg && sg[3] == cur_seg) {
                        // whole group inside the current segment (segment ids are non-decreasing
                        // between the head and tail padding, which carries -1)
#pragma unroll
                        for (int k = 0; k < 4; ++k)
#pragma unroll
                            for (int v = 0; v < V; ++v) fma4(acc[v], av[k], b[k][v]);
                    } else {
#pragma unroll
                        for (int k = 0; k < 4; ++k) {
                            if (sg[k] >= 0) {                    // warp-uniform
                                if (sg[k] != cur_seg) {
                                    if (cur_seg >= 0) flush(cur_seg);
                                    cur_seg = sg[k];
#pragma unroll
                                    for (int v = 0; v < V; ++v) acc[v] = make_float4(0.f, 0.f, 0.f, 0.f);
                                }
#pragma unroll
                                for (int v = 0; v < V; ++v) fma4(acc[v], av[k], b[k][v]);
                            }
                        }
                    }
                    __syncwarp();
                    const int gf = gc + NG;
                    if (gf < num_groups) fetch(gf, cstep);
                    stream_commit();
                }
            }
        }
        if (cur_seg >= 0) flush(cur_seg);
        stream_wait<0>();

        // ---- empty rows (only consecutive-row mode can contain them) ----------
        if (kMode == kModeRows) {
            unsigned empties = __ballot_sync(0xffffffffu, lane < count && len == 0);
#pragma unroll
            for (int v = 0; v < V; ++v) acc[v] = make_float4(0.f, 0.f, 0.f, 0.f);
            while (empties) {
                const int j = __ffs(empties) - 1;
                empties &= empties - 1;
                flush(j);
            }
        }
        __syncwarp();
    }
}

// Launch helper. Requires N in {128,256,512}, B/C (and scratch) 16-byte aligned;
// kModeRows also needs colind/vals 16-byte aligned.
// total_nnz is only used by kModeRows (weight-balanced row ranges); pass < 0 when unknown.
template <int kMode>
inline int launch_csr_stream(const StreamArgs& a, cudaStream_t st, long long total_nnz = -1)
{
    if (a.num_items <= 0) return RA_OK;
    StreamArgs args = a;
    args.weight_per_warp = 0;
    const int V = a.N / 128;
    // short batches for chunks (up to 256 nonzeros each), full batches for rows
    args.segs_per_batch = (kMode == kModeChunks) ? 2 : 32;
    const long long batches = (a.num_items + args.segs_per_batch - 1) / args.segs_per_batch;
    const int smem = kStreamWarps * stream_warp_smem(V);
    const int ctas_per_sm = std::max(1, (220 * 1024) / (smem + 1024));
    // enough warps for several waves, at most 8 batches per warp
    const long long target_warps = (long long)sm_count() * ctas_per_sm * kStreamWarps * 6;
    long long bpw = batches / target_warps;
    if (bpw < 1) bpw = 1;
    if (bpw > 8) bpw = 8;
    args.batches_per_warp = (int)bpw;
    long long warps = (batches + bpw - 1) / bpw;
    if (kMode == kModeRows && total_nnz >= 0) {
        const long long total_w = total_nnz + a.num_items;
        long long wpw = (total_w + target_warps - 1) / target_warps;
        if (wpw < 128) wpw = 128;
        args.weight_per_warp = wpw;
        warps = (total_w + wpw - 1) / wpw + 1;      // +1: the last range is closed by num_items
    }
    const int ctas = (int)((warps + kStreamWarps - 1) / kStreamWarps);
#define RA_STREAM_LAUNCH(VV)                                                                   \
    do {                                                                                       \
        auto kern = csr_stream_kernel<VV, kMode>;                                              \
        static std::atomic<unsigned long long> configured{0};                                  \
        RA_CUDA_TRY(configure_once_per_device(configured, [&]() -> cudaError_t {               \
            cudaError_t e_ = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem); \
            if (e_ != cudaSuccess) return e_;                                                  \
            return cudaFuncSetAttribute(kern, cudaFuncAttributePreferredSharedMemoryCarveout, 100); \
        }));                                                                                   \
        kern<<<ctas, kStreamThreads, smem, st>>>(args);                                        \
    } while (0)
    if (V == 1) RA_STREAM_LAUNCH(1);
    else if (V == 2) RA_STREAM_LAUNCH(2);
    else if (V == 4) RA_STREAM_LAUNCH(4);
    else { set_error("csr stream kernel: unsupported N=%d", a.N); return RA_ERR_UNSUPPORTED; }
#undef RA_STREAM_LAUNCH
    RA_KERNEL_CHECK();
    return RA_OK;
}

inline bool stream_width_ok(int N) { return N == 128 || N == 256 || N == 512; }

// ===========================================================================
// Group-aligned variant for listed rows and chunks, N in {32, 64, 128, 256, 512}.
//
// Every segment is padded (in stream coordinates only) to a multiple of 4
// elements, so a ring group of 4 B rows never straddles two segments: the
// consumer needs no running-segment bookkeeping, and for narrow rows the four
// elements of a group are multiplied in parallel by 32/L lane groups
// (L = N/4 lanes cover one B row; N=64: two rows per copy instruction, N=32:
// four) whose partial rows are combined with shuffle-xor when the segment ends.
// One segment search per lane and step instead of one per element.
// ===========================================================================
template <int L, int V>
struct AlignedCfg {
    static constexpr int kSub      = 32 / L;               // lane groups = rows per copy instruction
    static constexpr int kRowBytes = 16 * L * V;           // one B row
    static constexpr int kSlots    = (L == 32) ? 16 : (L == 16 ? 32 : 64);
    static constexpr int kGroups   = kSlots / 4;
    static constexpr int kWarpSmem = kSlots * kRowBytes + 1024;   // ring + per-step group table
};

template <int L, int V, int kMode>
__global__ void __launch_bounds__(kStreamThreads, (V == 1) ? 6 : ((V == 2) ? 3 : 1))
csr_stream_aligned_kernel(StreamArgs a)
{
    using Cfg = AlignedCfg<L, V>;
    constexpr int kSub = Cfg::kSub;
    constexpr int NG = Cfg::kGroups;
    constexpr int kRowBytes = Cfg::kRowBytes;
    static_assert(L == 32 || V == 1, "wide rows use all 32 lanes");
    extern __shared__ __align__(16) unsigned char smem[];

    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    const int sub = lane / L;                      // which of the kSub rows of a copy this lane serves
    const int sl = lane % L;
    unsigned char* ring_ptr = smem + warp * Cfg::kWarpSmem;
    const unsigned ring = (unsigned)__cvta_generic_to_shared(ring_ptr);
    float4* table = reinterpret_cast<float4*>(ring_ptr + Cfg::kSlots * kRowBytes);   // [32][2]: values, code
    long long gwarp = (long long)blockIdx.x * kStreamWarps + warp;
    const int N = a.N;
    // warp-uniform: does this warp walk chunks or listed rows?
    bool is_chunk = (kMode == kModeChunks);
    int spb = a.segs_per_batch;
    int bpw = a.batches_per_warp;
    long long num_items = a.num_items;
    if (kMode == kModeFused) {
        if (gwarp < a.chunk_warps) {
            is_chunk = true; spb = 2; bpw = a.chunk_batches_per_warp; num_items = a.num_chunks;
        } else {
            gwarp -= a.chunk_warps;
        }
    }
    const unsigned char* Bbytes = reinterpret_cast<const unsigned char*>(a.B);
    const size_t b_row_bytes = (size_t)N * 4;

    auto load_meta = [&](long long first, long long limit, int& s, int& e, float*& dst) {
        s = 0; e = 0; dst = nullptr;
        const long long it = first + lane;
        if (lane < spb && it < limit) {
            if (is_chunk) {
                const unsigned tag = (unsigned)__ldg(a.chunk_rows + it);
                const int row = (int)(tag & ~kStreamSoleFlag);
                s = __ldg(a.chunk_starts + it);
                e = min(s + kStreamChunk, __ldg(a.rowptr + row + 1));
                const int slot = __ldg(a.chunk_slot + it);
                dst = (slot < 0) ? a.C + (size_t)row * N : a.scratch + (size_t)slot * N;
            } else {
                const int row = a.row_ids ? __ldg(a.row_ids + it) : (int)it;
                s = __ldg(a.rowptr + row);
                e = __ldg(a.rowptr + row + 1);
                dst = a.C + (size_t)row * N;
            }
        }
    };

    long long it_lo, it_hi;
    if (kMode == kModeListed && a.weight_per_warp > 0) {
        // consecutive rows dealt out by weight = nonzeros + rows (a row is never split), so a
        // run of hub rows does not end up in one warp
        const int base = __ldg(a.rowptr);
        auto weight_lower_bound = [&](long long target) -> long long {
            long long lo = 0, hi = num_items;       // smallest r with rowptr[r]-rowptr[0]+r >= target
            while (lo < hi) {
                const long long mid = (lo + hi) >> 1;
                if ((long long)(__ldg(a.rowptr + mid) - base) + mid < target) lo = mid + 1; else hi = mid;
            }
            return lo;
        };
        it_lo = weight_lower_bound(gwarp * a.weight_per_warp);
        it_hi = weight_lower_bound((gwarp + 1) * a.weight_per_warp);
        if (gwarp == (long long)gridDim.x * kStreamWarps - 1) it_hi = num_items;
    } else {
        it_lo = gwarp * bpw * spb;
        it_hi = min(num_items, it_lo + (long long)bpw * spb);
    }
    if (it_lo >= it_hi) return;
    int s_n, e_n; float* dst_n;
    load_meta(it_lo, it_hi, s_n, e_n, dst_n);

    struct GSet { int c[4]; float v[4]; int code; };   // one group per lane

#pragma unroll 1
    for (long long first = it_lo; first < it_hi; first += spb) {
        const int count = (int)min((long long)spb, it_hi - first);
        const int s = s_n, e = e_n;
        float* dst = dst_n;
        if (first + spb < it_hi) load_meta(first + spb, it_hi, s_n, e_n, dst_n);   // prefetch

        const int len = e - s;
        const int plen = (len + 3) & ~3;                   // padded length
        int inc = plen;
#pragma unroll
        for (int off = 1; off < 32; off <<= 1) {
            const int y = __shfl_up_sync(0xffffffffu, inc, off);
            if (lane >= off) inc += y;
        }
        const int seg_begin = (lane < count) ? (inc - plen) : 0x7fffffff;
        const int total = __shfl_sync(0xffffffffu, inc, 31);
        const int num_groups = total >> 2;

        // group gi (coordinates 4gi..4gi+3) -> columns, values, code; code = -1 for no group,
        // else segment | valid count << 8 | last-group-of-segment << 12
        auto load_set = [&](int step) -> GSet {
            GSet g;
            const int x = step * 128 + 4 * lane;
            int j = 0;
#pragma unroll
            for (int st = 16; st > 0; st >>= 1) {
                const int cand = j + st;
                const int bv = __shfl_sync(0xffffffffu, seg_begin, cand & 31);
                if (cand < count && bv <= x) j = cand;
            }
            const int sj = __shfl_sync(0xffffffffu, s, j);
            const int lj = __shfl_sync(0xffffffffu, len, j);
            const int bj = __shfl_sync(0xffffffffu, seg_begin, j);
            const int off = x - bj;
            const bool have = x < total;
            const int nvalid = have ? min(4, lj - off) : 0;
            g.code = have ? (j | (nvalid << 8) | ((off + 4 >= lj) ? (1 << 12) : 0)) : -1;
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                g.c[k] = -1; g.v[k] = 0.f;
                if (k < nvalid) {
                    g.c[k] = __ldcs(a.colind + sj + off + k);
                    g.v[k] = __ldcs(a.vals + sj + off + k);
                }
            }
            return g;
        };
        auto publish = [&](const GSet& g) {
            table[2 * lane] = make_float4(g.v[0], g.v[1], g.v[2], g.v[3]);
            table[2 * lane + 1] = make_float4(__int_as_float(g.code), 0.f, 0.f, 0.f);
        };

        GSet cur = load_set(0);
        GSet nxt;
        if (total > 128) nxt = load_set(1);
        else { nxt.code = -1;
#pragma unroll
               for (int k = 0; k < 4; ++k) { nxt.c[k] = -1; nxt.v[k] = 0.f; } }
        __syncwarp();
        publish(cur);
        __syncwarp();

        // copies of one group: 4/kSub instructions, each moving kSub rows
        auto fetch = [&](int gf, int consume_step) {
            const bool use_cur = (gf >> 5) == consume_step;
            const int src = gf & 31;
            int cols[4];
            if (use_cur) {
#pragma unroll
                for (int k = 0; k < 4; ++k) cols[k] = __shfl_sync(0xffffffffu, cur.c[k], src);
            } else {
#pragma unroll
                for (int k = 0; k < 4; ++k) cols[k] = __shfl_sync(0xffffffffu, nxt.c[k], src);
            }
            const unsigned slot0 = ring + (unsigned)(((gf * 4) % Cfg::kSlots) * kRowBytes) + sl * 16;
#pragma unroll
            for (int i = 0; i < 4 / kSub; ++i) {
                // element handled by this lane group in copy i
                int col;
                if (kSub == 1) col = cols[i];
                else if (kSub == 2) col = sub ? cols[2 * i + 1] : cols[2 * i];
                else col = (sub == 0) ? cols[0] : (sub == 1) ? cols[1] : (sub == 2) ? cols[2] : cols[3];
                const int el = i * kSub + sub;
                if (col >= 0) {
                    const unsigned char* g = Bbytes + (size_t)col * b_row_bytes + sl * 16;
#pragma unroll
                    for (int v = 0; v < V; ++v)
                        stream_cp_async_16(slot0 + el * kRowBytes + v * 512, g + v * 512);
                }
            }
        };

#pragma unroll 1
        for (int gf = 0; gf < NG; ++gf) {
            if (gf < num_groups) fetch(gf, 0);
            stream_commit();
        }

        float4 acc[V];
#pragma unroll
        for (int v = 0; v < V; ++v) acc[v] = make_float4(0.f, 0.f, 0.f, 0.f);

#pragma unroll 1
        for (int g0 = 0; g0 < num_groups; g0 += NG) {
            if (g0 > 0 && (g0 & 31) == 0) {
                cur = nxt;
                __syncwarp();
                publish(cur);
                const int step = (g0 >> 5) + 1;
                if (step * 128 < total) nxt = load_set(step);
            }
            const int cstep = g0 >> 5;
#pragma unroll
            for (int jg = 0; jg < NG; ++jg) {
                const int gc = g0 + jg;
                if (gc < num_groups) {                           // warp-uniform
                    stream_wait<NG - 1>();
                    __syncwarp();
                    const float4 vals4 = table[2 * (gc & 31)];
                    const int code = __float_as_int(table[2 * (gc & 31) + 1].x);
                    const int nvalid = (code >> 8) & 15;
                    const unsigned char* slot0 = ring_ptr + ((gc * 4) % Cfg::kSlots) * kRowBytes + sl * 16;
                    const float va4[4] = {vals4.x, vals4.y, vals4.z, vals4.w};
#pragma unroll
                    for (int i = 0; i < 4 / kSub; ++i) {
                        const int el = i * kSub + sub;
                        float av;
                        if (kSub == 1) av = va4[i];
                        else if (kSub == 2) av = sub ? va4[2 * i + 1] : va4[2 * i];
                        else av = (sub == 0) ? va4[0] : (sub == 1) ? va4[1] : (sub == 2) ? va4[2] : va4[3];
                        if (el < nvalid) {
#pragma unroll
                            for (int v = 0; v < V; ++v) {
                                const float4 b = *reinterpret_cast<const float4*>(slot0 + el * kRowBytes + v * 512);
                                fma4(acc[v], av, b);
                            }
                        }
                    }
                    if (code & (1 << 12)) {                      // last group of its segment: write the row
                        const int seg = code & 255;
#pragma unroll
                        for (int off = L; off < 32; off <<= 1) {
#pragma unroll
                            for (int v = 0; v < V; ++v) {
                                acc[v].x += __shfl_xor_sync(0xffffffffu, acc[v].x, off);
                                acc[v].y += __shfl_xor_sync(0xffffffffu, acc[v].y, off);
                                acc[v].z += __shfl_xor_sync(0xffffffffu, acc[v].z, off);
                                acc[v].w += __shfl_xor_sync(0xffffffffu, acc[v].w, off);
                            }
                        }
                        const unsigned long long d =
                            ((unsigned long long)__shfl_sync(0xffffffffu, (unsigned)((unsigned long long)dst >> 32), seg) << 32) |
                            (unsigned long long)__shfl_sync(0xffffffffu, (unsigned)((unsigned long long)dst & 0xffffffffu), seg);
                        if (lane < L) {
                            float4* out = reinterpret_cast<float4*>(d) + lane;
#pragma unroll
                            for (int v = 0; v < V; ++v) st_stream_float4(out + v * 32, acc[v]);
                        }
#pragma unroll
                        for (int v = 0; v < V; ++v) acc[v] = make_float4(0.f, 0.f, 0.f, 0.f);
                    }
                    __syncwarp();
                    const int gf = gc + NG;
                    if (gf < num_groups) fetch(gf, cstep);
                    stream_commit();
                }
            }
        }
        stream_wait<0>();
        // rows without nonzeros never enter the stream: write their zeros here
        // (consecutive-row use of the listed mode; plan lists hold no empty rows)
        if (kMode != kModeChunks && !is_chunk) {
            unsigned empties = __ballot_sync(0xffffffffu, lane < count && len == 0);
            while (empties) {
                const int j = __ffs(empties) - 1;
                empties &= empties - 1;
                const unsigned long long d =
                    ((unsigned long long)__shfl_sync(0xffffffffu, (unsigned)((unsigned long long)dst >> 32), j) << 32) |
                    (unsigned long long)__shfl_sync(0xffffffffu, (unsigned)((unsigned long long)dst & 0xffffffffu), j);
                if (lane < L) {
                    float4* out = reinterpret_cast<float4*>(d) + lane;
#pragma unroll
                    for (int v = 0; v < V; ++v) st_stream_float4(out + v * 32, make_float4(0.f, 0.f, 0.f, 0.f));
                }
            }
        }
        __syncwarp();
    }
}

inline bool stream_aligned_width_ok(int N) { return N == 32 || N == 64 || N == 128 || N == 256 || N == 512; }

// kMode: kModeListed (row_ids may be null = consecutive rows), kModeChunks, or kModeFused
// (num_items listed rows + num_chunks chunks in one launch).
// total_nnz >= 0 with kModeListed and null row_ids: consecutive rows are dealt to warps by
// weight (nonzeros + rows) instead of by count.
template <int kMode>
inline int launch_csr_stream_aligned(const StreamArgs& a, cudaStream_t st, long long total_nnz = -1)
{
    if (a.num_items <= 0) return RA_OK;
    StreamArgs args = a;
    args.weight_per_warp = 0;
    const bool by_weight = (kMode == kModeListed) && a.row_ids == nullptr && total_nnz >= 0;
    // rows: 32 per batch, fewer when the matrix is too small to fill the GPU that way
    long long spb = a.num_items / ((long long)sm_count() * 16);
    spb = std::max<long long>(2, std::min<long long>(32, spb));
    args.segs_per_batch = (kMode == kModeChunks) ? 2 : (int)spb;
    const long long batches = (a.num_items + args.segs_per_batch - 1) / args.segs_per_batch;
    const long long chunk_batches = (kMode == kModeFused) ? (a.num_chunks + 1) / 2 : 0;
#define RA_ALIGNED_LAUNCH(LL, VV)                                                              \
    do {                                                                                       \
        using Cfg = AlignedCfg<LL, VV>;                                                        \
        const int smem = kStreamWarps * Cfg::kWarpSmem;                                        \
        const int ctas_per_sm = std::max(1, std::min(6, (220 * 1024) / (smem + 1024)));        \
        const long long target_warps = (long long)sm_count() * ctas_per_sm * kStreamWarps * 6; \
        long long bpw = batches / target_warps;                                                \
        if (bpw < 1) bpw = 1;                                                                  \
        if (bpw > 8) bpw = 8;                                                                  \
        args.batches_per_warp = (int)bpw;                                                      \
        long long warps = (batches + bpw - 1) / bpw;                                           \
        if (by_weight) {                                                                       \
            const long long total_w = total_nnz + a.num_items;                                 \
            long long wpw = (total_w + warps - 1) / warps;                                     \
            if (wpw < 1) wpw = 1;                                                              \
            args.weight_per_warp = wpw;                                                        \
            warps = (total_w + wpw - 1) / wpw + 1;   /* the last range is closed by num_items */ \
        }                                                                                      \
        int ctas = (int)((warps + kStreamWarps - 1) / kStreamWarps);                           \
        if (kMode == kModeFused) {               /* whole CTAs of chunk warps come first */     \
            long long cbpw = chunk_batches / target_warps;                                     \
            if (cbpw < 1) cbpw = 1;                                                            \
            if (cbpw > 8) cbpw = 8;                                                            \
            const long long cwarps = (chunk_batches + cbpw - 1) / cbpw;                        \
            const int cctas = (int)((cwarps + kStreamWarps - 1) / kStreamWarps);               \
            args.chunk_batches_per_warp = (int)cbpw;                                           \
            args.chunk_warps = (long long)cctas * kStreamWarps;                                \
            ctas += cctas;                                                                     \
        }                                                                                      \
        auto kern = csr_stream_aligned_kernel<LL, VV, kMode>;                                  \
        static std::atomic<unsigned long long> configured{0};                                  \
        RA_CUDA_TRY(configure_once_per_device(configured, [&]() -> cudaError_t {               \
            cudaError_t e_ = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem); \
            if (e_ != cudaSuccess) return e_;                                                  \
            return cudaFuncSetAttribute(kern, cudaFuncAttributePreferredSharedMemoryCarveout, 100); \
        }));                                                                                   \
        kern<<<ctas, kStreamThreads, smem, st>>>(args);                                        \
    } while (0)
    switch (a.N) {
        case 32:  RA_ALIGNED_LAUNCH(8, 1); break;
        case 64:  RA_ALIGNED_LAUNCH(16, 1); break;
        case 128: RA_ALIGNED_LAUNCH(32, 1); break;
        case 256: RA_ALIGNED_LAUNCH(32, 2); break;
        case 512: RA_ALIGNED_LAUNCH(32, 4); break;
        default: set_error("aligned stream kernel: unsupported N=%d", a.N); return RA_ERR_UNSUPPORTED;
    }
#undef RA_ALIGNED_LAUNCH
    RA_KERNEL_CHECK();
    return RA_OK;
}


}  // namespace ra
