// Long-row chunks of ZERO_OVERHEAD_CSR with a short instruction path.
//
// A chunk is a run of at most 256 consecutive nonzeros of one row (rows longer than 64
// nonzeros; the chunk list of the plan, csr/ra_zero_overhead.cu:349-374). The general
// streaming engine (csr_stream.cuh) treats chunks like any batch of segments - segment search,
// per-group tables, flush checks - and spends about 20 warp instructions per nonzero, which is
// what bounds it on matrices whose nonzeros sit mostly in long rows (an R-MAT graph keeps 86 %
// of them there). A chunk needs none of that: one destination, one contiguous range. Here a
// warp
//   1. copies the chunk's columns and values to shared memory (coalesced 4-byte loads, padded
//      to a whole group with the last column and zero values, so the loops carry no
//      predicates),
//   2. streams the B rows through its ring with 16-byte cp.async - at N = 64 one copy
//      instruction moves two rows, at N = 32 four - three to seven groups ahead of the
//      multiply, the column read from shared memory by a broadcast load,
//   3. multiplies group by group (one 128-bit shared load + two packed FMAs per row and lane),
//      combines the lane groups by shuffle and writes the row (a sole chunk) or the scratch
//      slot (a chunk of a multi-chunk row, merged later in chunk order).
// Replaces zo_chunk_vec4_kernel (csr/ra_zero_overhead.cu:226-268) for N in {32,64,128,256,512}.
#pragma once

#include "csr_stream.cuh"

namespace ra {

template <int L, int V>
struct ChunkCfg {
    static constexpr int kSub       = 32 / L;                // rows per copy instruction
    static constexpr int kRowBytes  = 16 * L * V;
    static constexpr int kGroupRows = 4 * kSub;              // 4 copy instructions per group
    static constexpr int kGroups    = (V == 4) ? 2 : 4;      // groups in the ring
    static constexpr int kSlots     = kGroups * kGroupRows;
    static constexpr int kListInts  = 256 + 16;              // columns / values of one chunk, padded
    static constexpr int kWarpSmem  = kSlots * kRowBytes + 2 * kListInts * 4;
};

template <int L, int V>
__global__ void __launch_bounds__(kStreamThreads)
zo_chunk_lean_kernel(const int* __restrict__ rowptr, const int* __restrict__ colind,
                     const float* __restrict__ vals, const float* __restrict__ B,
                     float* __restrict__ C, float* __restrict__ scratch,
                     const int* __restrict__ chunk_rows, const int* __restrict__ chunk_starts,
                     const int* __restrict__ chunk_slot, int num_chunks, int chunks_per_warp, int N)
{
    using Cfg = ChunkCfg<L, V>;
    constexpr int kSub = Cfg::kSub, NG = Cfg::kGroups, GR = Cfg::kGroupRows, kRowBytes = Cfg::kRowBytes;
    extern __shared__ __align__(16) unsigned char smem[];

    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    const int sub = lane / L, sl = lane % L;
    unsigned char* ring_ptr = smem + (size_t)warp * Cfg::kWarpSmem;
    const unsigned ring = (unsigned)__cvta_generic_to_shared(ring_ptr);
    int* colS = reinterpret_cast<int*>(ring_ptr + Cfg::kSlots * kRowBytes);
    float* valS = reinterpret_cast<float*>(colS + Cfg::kListInts);
    const unsigned char* Bbytes = reinterpret_cast<const unsigned char*>(B);
    const size_t b_row_bytes = (size_t)N * 4;

    const long long gwarp = (long long)blockIdx.x * kStreamWarps + warp;
    const long long c_lo = gwarp * chunks_per_warp;
    const long long c_hi = min((long long)num_chunks, c_lo + chunks_per_warp);

#pragma unroll 1
    for (long long c = c_lo; c < c_hi; ++c) {
        const unsigned tag = (unsigned)__ldg(chunk_rows + c);
        const int row = (int)(tag & ~kStreamSoleFlag);
        const int s = __ldg(chunk_starts + c);
        const int e = min(s + kStreamChunk, __ldg(rowptr + row + 1));
        const int slot = __ldg(chunk_slot + c);
        const int len = e - s;
        const int num_groups = (len + GR - 1) / GR;
        const int padded = num_groups * GR;

        // ---- 1. columns / values of the chunk -> shared memory ----
        __syncwarp();                                   // the previous chunk's reads of the lists are done
#pragma unroll
        for (int k = 0; k < 8; ++k) {            // padded <= 256
            const int idx = k * 32 + lane;
            if (idx < padded) {
                const int p = s + min(idx, len - 1);    // padding repeats the last column ...
                colS[idx] = __ldcs(colind + p);
                valS[idx] = (idx < len) ? __ldcs(vals + p) : 0.f;     // ... with a zero value
            }
        }
        __syncwarp();

        // ---- 2./3. gather ring + multiply ----
        auto fetch = [&](int gf) {
            const int first = gf * GR;
            const unsigned slot0 = ring + (unsigned)(((gf % NG) * GR) * kRowBytes) + sl * 16;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int r = i * kSub + sub;            // row of the group served by this lane group
                const int col = colS[first + r];
                const unsigned char* g = Bbytes + (size_t)col * b_row_bytes + sl * 16;
#pragma unroll
                for (int v = 0; v < V; ++v) stream_cp_async_16(slot0 + r * kRowBytes + v * 512, g + v * 512);
            }
        };
#pragma unroll 1
        for (int gf = 0; gf < NG - 1; ++gf) {
            if (gf < num_groups) fetch(gf);
            stream_commit();
        }
        float4 acc[V];
#pragma unroll
        for (int v = 0; v < V; ++v) acc[v] = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 1
        for (int gc = 0; gc < num_groups; ++gc) {
            // refill the slot consumed in the previous iteration, then wait for group gc
            if (gc + NG - 1 < num_groups) fetch(gc + NG - 1);
            stream_commit();
            stream_wait<NG - 1>();
            __syncwarp();
            const unsigned char* slot0 = ring_ptr + ((gc % NG) * GR) * kRowBytes + sl * 16;
            const int first = gc * GR;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int r = i * kSub + sub;
                const float av = valS[first + r];
#pragma unroll
                for (int v = 0; v < V; ++v) {
                    const float4 b = *reinterpret_cast<const float4*>(slot0 + r * kRowBytes + v * 512);
                    fma4(acc[v], av, b);
                }
            }
            __syncwarp();                                // all lanes are done with the slot before it is refilled
        }
        stream_wait<0>();

        // ---- combine the lane groups, write the row or the scratch slot ----
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
        if (lane < L) {
            float4* out = reinterpret_cast<float4*>((slot < 0) ? C + (size_t)row * N : scratch + (size_t)slot * N) + lane;
            if (slot < 0) {
#pragma unroll
                for (int v = 0; v < V; ++v) st_stream_float4(out + v * 32, acc[v]);
            } else {
#pragma unroll
                for (int v = 0; v < V; ++v) out[v * 32] = acc[v];
            }
        }
    }
}

// Register variant of the chunk kernel: the B rows go straight from L2 into registers
// (128-bit read-only loads) instead of through a shared-memory ring, so every gathered byte
// crosses the SM's load/store data path once instead of twice (ring fill + ring read) - the
// ring kernels top out near 9 TB/s of gathered bytes at 256-byte rows, about half the data
// path of an SM is spent on the second crossing. A lane keeps U rows of the next group in
// flight while it multiplies the U rows of the current one; the columns and values of the chunk
// still sit in shared memory (step 1 of the ring kernel) and are read by broadcast loads.
template <int L, int V, int U>
__global__ void __launch_bounds__(kStreamThreads)
zo_chunk_reg_kernel(const int* __restrict__ rowptr, const int* __restrict__ colind,
                    const float* __restrict__ vals, const float* __restrict__ B,
                    float* __restrict__ C, float* __restrict__ scratch,
                    const int* __restrict__ chunk_rows, const int* __restrict__ chunk_starts,
                    const int* __restrict__ chunk_slot, int num_chunks, int chunks_per_warp, int N)
{
    constexpr int kSub = 32 / L;
    constexpr int GR = U * kSub;                               // rows per group
    constexpr int kListInts = 256 + 32;
    __shared__ int   colS_all[kStreamWarps][kListInts];
    __shared__ float valS_all[kStreamWarps][kListInts];

    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    const int sub = lane / L, sl = lane % L;
    int* colS = colS_all[warp];
    float* valS = valS_all[warp];
    const float4* B4 = reinterpret_cast<const float4*>(B);
    const int N4 = N >> 2;

    const long long gwarp = (long long)blockIdx.x * kStreamWarps + warp;
    const long long c_lo = gwarp * chunks_per_warp;
    const long long c_hi = min((long long)num_chunks, c_lo + chunks_per_warp);

#pragma unroll 1
    for (long long c = c_lo; c < c_hi; ++c) {
        const unsigned tag = (unsigned)__ldg(chunk_rows + c);
        const int row = (int)(tag & ~kStreamSoleFlag);
        const int s = __ldg(chunk_starts + c);
        const int e = min(s + kStreamChunk, __ldg(rowptr + row + 1));
        const int slot = __ldg(chunk_slot + c);
        const int len = e - s;
        const int num_groups = (len + GR - 1) / GR;
        const int padded = num_groups * GR;

        __syncwarp();
#pragma unroll
        for (int k = 0; k < 9; ++k) {                          // padded <= 256 + GR - 1 < 288
            const int idx = k * 32 + lane;
            if (idx < padded) {
                const int p = s + min(idx, len - 1);            // padding repeats the last column with a zero value
                colS[idx] = __ldcs(colind + p);
                valS[idx] = (idx < len) ? __ldcs(vals + p) : 0.f;
            }
        }
        __syncwarp();

        float4 cur[U][V], nxt[U][V];
        auto load_group = [&](int gidx, float4 (&dst)[U][V]) {
            const int first = gidx * GR;
#pragma unroll
            for (int i = 0; i < U; ++i) {
                const float4* brow = B4 + (size_t)colS[first + i * kSub + sub] * N4 + sl;
#pragma unroll
                for (int v = 0; v < V; ++v) dst[i][v] = ld_gather_float4(brow + v * 32);
            }
        };
        float4 acc[V];
#pragma unroll
        for (int v = 0; v < V; ++v) acc[v] = make_float4(0.f, 0.f, 0.f, 0.f);
        load_group(0, cur);
#pragma unroll 1
        for (int gc = 0; gc < num_groups; ++gc) {
            if (gc + 1 < num_groups) load_group(gc + 1, nxt);
            const int first = gc * GR;
#pragma unroll
            for (int i = 0; i < U; ++i) {
                const float av = valS[first + i * kSub + sub];
#pragma unroll
                for (int v = 0; v < V; ++v) fma4(acc[v], av, cur[i][v]);
            }
#pragma unroll
            for (int i = 0; i < U; ++i)
#pragma unroll
                for (int v = 0; v < V; ++v) cur[i][v] = nxt[i][v];
        }
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
        if (lane < L) {
            float4* out = reinterpret_cast<float4*>((slot < 0) ? C + (size_t)row * N : scratch + (size_t)slot * N) + lane;
            if (slot < 0) {
#pragma unroll
                for (int v = 0; v < V; ++v) st_stream_float4(out + v * 32, acc[v]);
            } else {
#pragma unroll
                for (int v = 0; v < V; ++v) out[v * 32] = acc[v];
            }
        }
    }
}

inline int launch_zo_chunks_reg(const int* rowptr, const int* colind, const float* vals, const float* B,
                                float* C, float* scratch, const int* chunk_rows, const int* chunk_starts,
                                const int* chunk_slot, int num_chunks, int N, cudaStream_t st)
{
    if (num_chunks <= 0) return RA_OK;
    const long long warps_wave = (long long)sm_count() * 8 * kStreamWarps;
    const int cpw = (int)std::max<long long>(1, std::min<long long>(8, num_chunks / (warps_wave * 4)));
    const long long warps = ((long long)num_chunks + cpw - 1) / cpw;
    const int ctas = (int)((warps + kStreamWarps - 1) / kStreamWarps);
#define RA_CHUNK_REG(LL, VV, UU) zo_chunk_reg_kernel<LL, VV, UU><<<ctas, kStreamThreads, 0, st>>>( \
        rowptr, colind, vals, B, C, scratch, chunk_rows, chunk_starts, chunk_slot, num_chunks, cpw, N)
    switch (N) {
        case 32:  RA_CHUNK_REG(8, 1, 8); break;
        case 64:  RA_CHUNK_REG(16, 1, 8); break;
        case 128: RA_CHUNK_REG(32, 1, 8); break;
        case 256: RA_CHUNK_REG(32, 2, 4); break;
        case 512: RA_CHUNK_REG(32, 4, 2); break;
        default: set_error("register chunk kernel: unsupported N=%d", N); return RA_ERR_UNSUPPORTED;
    }
#undef RA_CHUNK_REG
    RA_KERNEL_CHECK();
    return RA_OK;
}

// Requires N in {32,64,128,256,512} and 16-byte aligned B, C, scratch.
inline int launch_zo_chunks_lean(const int* rowptr, const int* colind, const float* vals, const float* B,
                                 float* C, float* scratch, const int* chunk_rows, const int* chunk_starts,
                                 const int* chunk_slot, int num_chunks, int N, cudaStream_t st)
{
    if (num_chunks <= 0) return RA_OK;
#define RA_CHUNK_LAUNCH(LL, VV)                                                                \
    do {                                                                                       \
        using Cfg = ChunkCfg<LL, VV>;                                                          \
        const int smem = kStreamWarps * Cfg::kWarpSmem;                                        \
        const int ctas_per_sm = std::max(1, std::min(8, (220 * 1024) / (smem + 1024)));        \
        /* a few chunks per warp once the grid has several waves: amortises the warp start */  \
        const long long warps_wave = (long long)sm_count() * ctas_per_sm * kStreamWarps;       \
        int cpw = (int)std::max<long long>(1, std::min<long long>(8, num_chunks / (warps_wave * 4))); \
        const long long warps = ((long long)num_chunks + cpw - 1) / cpw;                       \
        const int ctas = (int)((warps + kStreamWarps - 1) / kStreamWarps);                     \
        auto kern = zo_chunk_lean_kernel<LL, VV>;                                              \
        static std::atomic<unsigned long long> configured{0};                                  \
        RA_CUDA_TRY(configure_once_per_device(configured, [&]() -> cudaError_t {               \
            cudaError_t e_ = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem); \
            if (e_ != cudaSuccess) return e_;                                                  \
            return cudaFuncSetAttribute(kern, cudaFuncAttributePreferredSharedMemoryCarveout, 100); \
        }));                                                                                   \
        kern<<<ctas, kStreamThreads, smem, st>>>(rowptr, colind, vals, B, C, scratch, chunk_rows, \
                                                 chunk_starts, chunk_slot, num_chunks, cpw, N); \
    } while (0)
    switch (N) {
        case 32:  RA_CHUNK_LAUNCH(8, 1); break;
        case 64:  RA_CHUNK_LAUNCH(16, 1); break;
        case 128: RA_CHUNK_LAUNCH(32, 1); break;
        case 256: RA_CHUNK_LAUNCH(32, 2); break;
        case 512: RA_CHUNK_LAUNCH(32, 4); break;
        default: set_error("lean chunk kernel: unsupported N=%d", N); return RA_ERR_UNSUPPORTED;
    }
#undef RA_CHUNK_LAUNCH
    RA_KERNEL_CHECK();
    return RA_OK;
}

}  // namespace ra
