// ZERO_OVERHEAD_CSR for sm_100a: degree-binned dispatch with the plan built on
// the device.
//
// Replaces make/run/free_ra_zero_overhead_plan (csr/ra_zero_overhead.cu:312-519).
// The plan lists have the contents and order of the reference plan:
//   small_row_ids = rows with 1-4 nnz, then 5-16, then 17-64, each ascending;
//   chunks        = for every row with > 64 nnz, in row order: one entry tagged
//                   (row | 0x80000000, rowptr[row]) if nnz <= 256, else one
//                   entry (row, rowptr[row] + 256*j) per 256-nnz chunk;
//   zero_row_ids  = empty rows and multi-chunk rows, ascending.
// A stable partition by bin (exclusive scans of the bin indicators) keeps the
// ascending row order inside each list, which is what the serial host loop of
// the reference produces (csr/ra_zero_overhead.cu:331-374).
//
// Run: (1) chunks: a sole chunk writes its C row, a chunk of a multi-chunk row
// writes its partial row to a scratch slot; (2) the small rows go through the
// CSR streaming engine via the bin-ordered id list - at N in {32,64,128,256,512}
// (1) and (2) are one launch whose first warps take the chunks; (3) one finish
// launch walks zero_row_ids and writes each listed row as the sum of its
// scratch slots in ascending chunk order (no slots = an empty row = zeros).
// The reference adds multi-chunk partials with fp32 atomicAdd in arbitrary
// order; here the merge order is fixed, so results are run-to-run identical.
#include "csr_engine.cuh"
#include "csr_stream.cuh"
#include "scan.cuh"
#include "zo_plan.cuh"

#include <cstdlib>
#include <mutex>
#include <string>
#include <vector>

namespace ra {

int launch_csr_rows(const int* rowptr, const int* colind, const float* vals,
                    const float* B, float* C, const int* row_ids, int num_rows,
                    int N, cudaStream_t st, long long total_nnz);

constexpr int kTiny = 4, kShort = 16, kMedium = 64, kChunk = 256;
constexpr unsigned kSoleFlag = 0x80000000u;
constexpr int kZoThreads = 256;

// ---- plan build -------------------------------------------------------------
// channel layout of the per-row indicator arrays (each M ints, then scanned)
enum { CH_TINY = 0, CH_SHORT, CH_MED, CH_ZERO, CH_CHUNKS, CH_SLOTS, CH_COUNT };

__global__ void __launch_bounds__(kZoThreads)
zo_classify_kernel(const int* __restrict__ rowptr, int M, int* __restrict__ ind, i64 stride,
                   int* __restrict__ stats /* [0]=max long nnz, [1]=empty rows */)
{
    int local_max = 0, local_empty = 0;
    for (i64 i = (i64)blockIdx.x * blockDim.x + threadIdx.x; i < M;
         i += (i64)gridDim.x * blockDim.x) {
        const int nnz = rowptr[i + 1] - rowptr[i];
        const bool is_long = nnz > kMedium;
        const bool multi = nnz > kChunk;
        const int nchunks = !is_long ? 0 : (multi ? (nnz + kChunk - 1) / kChunk : 1);
        ind[CH_TINY * stride + i]   = (nnz >= 1 && nnz <= kTiny);
        ind[CH_SHORT * stride + i]  = (nnz > kTiny && nnz <= kShort);
        ind[CH_MED * stride + i]    = (nnz > kShort && nnz <= kMedium);
        ind[CH_ZERO * stride + i]   = (nnz == 0) || multi;
        ind[CH_CHUNKS * stride + i] = nchunks;
        ind[CH_SLOTS * stride + i]  = multi ? nchunks : 0;
        if (is_long) local_max = max(local_max, nnz);
        local_empty += (nnz == 0);
    }
    if (local_max > 0) atomicMax(stats, local_max);
    if (local_empty > 0) atomicAdd(stats + 1, local_empty);
}

struct ZoTotals { int tiny, shrt, med, zero, chunks, slots; };

__global__ void __launch_bounds__(kZoThreads)
zo_scatter_kernel(const int* __restrict__ rowptr, int M, const int* __restrict__ off, i64 stride,
                  ZoTotals t, int* __restrict__ small_ids, int* __restrict__ chunk_rows,
                  int* __restrict__ chunk_starts, int* __restrict__ chunk_slot,
                  int* __restrict__ zero_ids, int* __restrict__ zero_slot_off)
{
    for (i64 i = (i64)blockIdx.x * blockDim.x + threadIdx.x; i < M;
         i += (i64)gridDim.x * blockDim.x) {
        const int start = rowptr[i];
        const int nnz = rowptr[i + 1] - start;
        if (nnz == 0) {
            const int z = off[CH_ZERO * stride + i];
            zero_ids[z] = (int)i;
            zero_slot_off[z] = off[CH_SLOTS * stride + i];
        } else if (nnz <= kTiny) {
            small_ids[off[CH_TINY * stride + i]] = (int)i;
        } else if (nnz <= kShort) {
            small_ids[t.tiny + off[CH_SHORT * stride + i]] = (int)i;
        } else if (nnz <= kMedium) {
            small_ids[t.tiny + t.shrt + off[CH_MED * stride + i]] = (int)i;
        } else if (nnz <= kChunk) {
            const int c = off[CH_CHUNKS * stride + i];
            chunk_rows[c] = (int)((unsigned)i | kSoleFlag);
            chunk_starts[c] = start;
            chunk_slot[c] = -1;
        } else {
            const int z = off[CH_ZERO * stride + i];
            const int slot0 = off[CH_SLOTS * stride + i];
            zero_ids[z] = (int)i;
            zero_slot_off[z] = slot0;
            const int c0 = off[CH_CHUNKS * stride + i];
            const int nch = (nnz + kChunk - 1) / kChunk;
            for (int j = 0; j < nch; ++j) {
                chunk_rows[c0 + j] = (int)i;
                chunk_starts[c0 + j] = start + j * kChunk;
                chunk_slot[c0 + j] = slot0 + j;
            }
        }
    }
    if (blockIdx.x == 0 && threadIdx.x == 0) zero_slot_off[t.zero] = t.slots;
}

// ---- run ----------------------------------------------------------------------
template <int L, int V, int Q, bool kVecA>
__global__ void __launch_bounds__(kZoThreads)
zo_chunk_kernel(const int* __restrict__ rowptr, const int* __restrict__ colind,
                const float* __restrict__ vals, const float* __restrict__ B,
                float* __restrict__ C, float* __restrict__ scratch,
                const int* __restrict__ chunk_rows, const int* __restrict__ chunk_starts,
                const int* __restrict__ chunk_slot, int num_chunks, int N)
{
    using E = RowEngine<L, V, Q, kVecA>;
    const int lane = threadIdx.x & 31;
    const i64 c = ((i64)blockIdx.x * kZoThreads + threadIdx.x) >> 5;
    if (c >= num_chunks) return;
    const unsigned tag = (unsigned)__ldg(chunk_rows + c);
    const int row = (int)(tag & ~kSoleFlag);
    const int s = __ldg(chunk_starts + c);
    const int e = min(s + kChunk, __ldg(rowptr + row + 1));
    const int slot = __ldg(chunk_slot + c);
    const int N4 = N >> 2;
    float4 acc[V];
#pragma unroll
    for (int v = 0; v < V; ++v) acc[v] = make_float4(0.f, 0.f, 0.f, 0.f);
    const AChunk first = E::load(colind, vals, E::first_base(s), e, lane);
    E::accumulate(colind, vals, reinterpret_cast<const float4*>(B), N4, s, e, lane, first, acc);
    E::reduce_groups(acc);
    float* dst = (slot < 0) ? C + (i64)row * N : scratch + (i64)slot * N;
    if (slot < 0) {
        E::store_row(reinterpret_cast<float4*>(dst), lane, acc);
    } else if (lane < L) {
#pragma unroll
        for (int v = 0; v < V; ++v) reinterpret_cast<float4*>(dst)[lane + v * L] = acc[v];
    }
}

__global__ void __launch_bounds__(kZoThreads)
zo_chunk_generic_kernel(const int* __restrict__ rowptr, const int* __restrict__ colind,
                        const float* __restrict__ vals, const float* __restrict__ B,
                        float* __restrict__ C, float* __restrict__ scratch,
                        const int* __restrict__ chunk_rows, const int* __restrict__ chunk_starts,
                        const int* __restrict__ chunk_slot, int num_chunks, int N)
{
    const int lane = threadIdx.x & 31;
    const i64 c = ((i64)blockIdx.x * kZoThreads + threadIdx.x) >> 5;
    if (c >= num_chunks) return;
    const unsigned tag = (unsigned)__ldg(chunk_rows + c);
    const int row = (int)(tag & ~kSoleFlag);
    const int s = __ldg(chunk_starts + c);
    const int e = min(s + kChunk, __ldg(rowptr + row + 1));
    const int slot = __ldg(chunk_slot + c);
    float* dst = (slot < 0) ? C + (i64)row * N : scratch + (i64)slot * N;
    for (int n0 = 0; n0 < N; n0 += 128) {
        float acc[4] = {0.f, 0.f, 0.f, 0.f};
        generic_accumulate_tile(colind, vals, B, N, s, e, lane, n0, acc);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int n = n0 + lane + 32 * j;
            if (n < N) dst[n] = acc[j];
        }
    }
}

// Listed rows (empty rows and multi-chunk rows): C[row,:] = sum of the row's scratch slots in
// ascending chunk order (no slots = an empty row = zeros). vec4: one thread per float4 of a row,
// so a 64-wide row takes 16 threads and a warp covers two rows; two slots in flight per thread.
__global__ void __launch_bounds__(kZoThreads)
zo_finish_kernel(const int* __restrict__ zero_ids, const int* __restrict__ zero_slot_off,
                 const float* __restrict__ scratch, float* __restrict__ C,
                 int num_zero, int N, int vec4)
{
    if (vec4) {
        const int N4 = N >> 2;
        const i64 total = (i64)num_zero * N4;
        const float4* s4 = reinterpret_cast<const float4*>(scratch);
        for (i64 idx = (i64)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (i64)gridDim.x * blockDim.x) {
            const int z = (int)(idx / N4);
            const int n4 = (int)(idx - (i64)z * N4);
            const int row = __ldg(zero_ids + z);
            const int o0 = __ldg(zero_slot_off + z);
            const int o1 = __ldg(zero_slot_off + z + 1);
            float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
            int o = o0;
            for (; o + 2 <= o1; o += 2) {
                const float4 p = __ldcs(s4 + (i64)o * N4 + n4), q = __ldcs(s4 + (i64)(o + 1) * N4 + n4);
                acc.x += p.x; acc.y += p.y; acc.z += p.z; acc.w += p.w;
                acc.x += q.x; acc.y += q.y; acc.z += q.z; acc.w += q.w;
            }
            if (o < o1) {
                const float4 p = __ldcs(s4 + (i64)o * N4 + n4);
                acc.x += p.x; acc.y += p.y; acc.z += p.z; acc.w += p.w;
            }
            st_stream_float4(reinterpret_cast<float4*>(C + (i64)row * N) + n4, acc);
        }
    } else {
        const int lane = threadIdx.x & 31;
        const i64 warps = ((i64)gridDim.x * kZoThreads) >> 5;
        for (i64 z = ((i64)blockIdx.x * kZoThreads + threadIdx.x) >> 5; z < num_zero; z += warps) {
            const int row = __ldg(zero_ids + z);
            const int o0 = __ldg(zero_slot_off + z);
            const int o1 = __ldg(zero_slot_off + z + 1);
            for (int n = lane; n < N; n += 32) {
                float acc = 0.f;
                for (int o = o0; o < o1; ++o) acc += scratch[(i64)o * N + n];
                C[(i64)row * N + n] = acc;
            }
        }
    }
}

}  // namespace ra

// ---- C ABI ----------------------------------------------------------------------

extern "C" int ra_zo_plan_destroy(RaZoPlan* p)
{
    if (!p) return RA_OK;
    cudaFree(p->d_small_row_ids);
    cudaFree(p->d_chunk_rows);
    cudaFree(p->d_chunk_starts);
    cudaFree(p->d_chunk_slot);
    cudaFree(p->d_zero_row_ids);
    cudaFree(p->d_zero_slot_off);
    cudaFree(p->d_scratch);
    delete p;
    return RA_OK;
}

namespace {
struct DevBuf {   // frees on scope exit
    void* p = nullptr;
    ~DevBuf() { if (p) cudaFree(p); }
};
}

extern "C" int ra_zo_plan_create(const int32_t* rowptr, int rowptr_on_device, int M, int K,
                                 void* stream, RaZoPlan** out)
{
    using namespace ra;
    RA_REQUIRE(out != nullptr, RA_ERR_INVALID_ARG, "ra_zo_plan_create: out is null");
    *out = nullptr;
    RA_REQUIRE(M >= 0 && K >= 0, RA_ERR_INVALID_ARG, "ra_zo_plan_create: negative size");
    RA_REQUIRE(rowptr != nullptr || M == 0, RA_ERR_INVALID_ARG, "ra_zo_plan_create: rowptr is null");
    cudaStream_t st = static_cast<cudaStream_t>(stream);

    RaZoPlan* p = new RaZoPlan();
    p->M = M; p->K = K;
    if (M == 0) { *out = p; return RA_OK; }

    DevBuf rp_copy, ind_buf, tmp_buf, max_buf;
    const int* d_rowptr = rowptr;
    auto fail = [&](int code) { ra_zo_plan_destroy(p); return code; };
#define ZO_TRY(expr) do { cudaError_t _e = (expr); if (_e != cudaSuccess) { \
        ra::set_error("%s failed at %s:%d: %s", #expr, __FILE__, __LINE__, cudaGetErrorString(_e)); \
        return fail(RA_ERR_CUDA); } } while (0)

    if (!rowptr_on_device) {
        ZO_TRY(cudaMalloc(&rp_copy.p, sizeof(int) * ((size_t)M + 1)));
        ZO_TRY(cudaMemcpyAsync(rp_copy.p, rowptr, sizeof(int) * ((size_t)M + 1),
                               cudaMemcpyHostToDevice, st));
        d_rowptr = static_cast<const int*>(rp_copy.p);
    }
    const i64 stride = (i64)M + 1;     // each channel: M indicators -> M+1 offsets
    ZO_TRY(cudaMalloc(&ind_buf.p, sizeof(int) * (size_t)(stride * CH_COUNT)));
    ZO_TRY(cudaMalloc(&tmp_buf.p, sizeof(int) * (size_t)scan_tmp_ints(M)));
    ZO_TRY(cudaMalloc(&max_buf.p, 2 * sizeof(int)));
    ZO_TRY(cudaMemsetAsync(max_buf.p, 0, 2 * sizeof(int), st));
    int* ind = static_cast<int*>(ind_buf.p);

    const int grid = (int)std::min<i64>(((i64)M + kZoThreads - 1) / kZoThreads, (i64)sm_count() * 16);
    zo_classify_kernel<<<grid, kZoThreads, 0, st>>>(d_rowptr, M, ind, stride,
                                                    static_cast<int*>(max_buf.p));
    ZO_TRY(cudaGetLastError());
    for (int ch = 0; ch < CH_COUNT; ++ch) {
        ZO_TRY(exclusive_scan_i32(ind + ch * stride, ind + ch * stride, M,
                                  static_cast<int*>(tmp_buf.p), st));
    }
    int totals[CH_COUNT];
    for (int ch = 0; ch < CH_COUNT; ++ch) {
        ZO_TRY(cudaMemcpyAsync(&totals[ch], ind + ch * stride + M, sizeof(int),
                               cudaMemcpyDeviceToHost, st));
    }
    int stats[2] = {0, 0};
    ZO_TRY(cudaMemcpyAsync(stats, max_buf.p, 2 * sizeof(int), cudaMemcpyDeviceToHost, st));
    ZO_TRY(cudaStreamSynchronize(st));
    const int max_long_nnz = stats[0];

    ZoTotals t{totals[CH_TINY], totals[CH_SHORT], totals[CH_MED],
               totals[CH_ZERO], totals[CH_CHUNKS], totals[CH_SLOTS]};
    p->num_tiny = t.tiny; p->num_short = t.shrt; p->num_medium = t.med;
    p->num_small = t.tiny + t.shrt + t.med;
    p->num_chunks = t.chunks;
    p->num_zero_rows = t.zero;
    p->num_slots = t.slots;
    p->max_long_chunks = (max_long_nnz + kChunk - 1) / kChunk;

    auto alloc_ints = [&](int** ptr, size_t n) -> cudaError_t {
        if (n == 0) { *ptr = nullptr; return cudaSuccess; }
        return cudaMalloc(reinterpret_cast<void**>(ptr), n * sizeof(int));
    };
    ZO_TRY(alloc_ints(&p->d_small_row_ids, (size_t)p->num_small));
    ZO_TRY(alloc_ints(&p->d_chunk_rows, (size_t)p->num_chunks));
    ZO_TRY(alloc_ints(&p->d_chunk_starts, (size_t)p->num_chunks));
    ZO_TRY(alloc_ints(&p->d_chunk_slot, (size_t)p->num_chunks));
    ZO_TRY(alloc_ints(&p->d_zero_row_ids, (size_t)p->num_zero_rows));
    ZO_TRY(alloc_ints(&p->d_zero_slot_off, (size_t)p->num_zero_rows + 1));

    zo_scatter_kernel<<<grid, kZoThreads, 0, st>>>(
        d_rowptr, M, ind, stride, t, p->d_small_row_ids, p->d_chunk_rows, p->d_chunk_starts,
        p->d_chunk_slot, p->d_zero_row_ids, p->d_zero_slot_off);
    ZO_TRY(cudaGetLastError());

    p->num_empty = stats[1];
    p->num_long = M - p->num_small - p->num_empty;
    ZO_TRY(cudaStreamSynchronize(st));   // temporaries are freed on return
#undef ZO_TRY
    *out = p;
    return RA_OK;
}

extern "C" int ra_zo_plan_info(const RaZoPlan* p, RaZoInfo* out)
{
    using namespace ra;
    RA_REQUIRE(p && out, RA_ERR_INVALID_ARG, "ra_zo_plan_info: null argument");
    out->M = p->M; out->K = p->K;
    out->num_tiny = p->num_tiny; out->num_short = p->num_short; out->num_medium = p->num_medium;
    out->num_long = p->num_long; out->num_empty = p->num_empty;
    out->num_small = p->num_small; out->num_chunks = p->num_chunks;
    out->num_zero_rows = p->num_zero_rows; out->max_long_chunks = p->max_long_chunks;
    // same accounting as the reference: the four published lists only
    out->plan_bytes = (int64_t)sizeof(int) * ((int64_t)p->num_small + 2LL * p->num_chunks +
                                              (int64_t)p->num_zero_rows);
    out->d_small_row_ids = p->d_small_row_ids;
    out->d_chunk_rows = p->d_chunk_rows;
    out->d_chunk_starts = p->d_chunk_starts;
    out->d_zero_row_ids = p->d_zero_row_ids;
    return RA_OK;
}

namespace ra {

template <int L, int V, int Q>
static void launch_chunks(const RaZoPlan* p, const int* rowptr, const int* colind,
                          const float* vals, const float* B, float* C, int N, bool vec_a,
                          cudaStream_t st)
{
    const int blocks = (int)(((i64)p->num_chunks * 32 + kZoThreads - 1) / kZoThreads);
    if (vec_a) {
        zo_chunk_kernel<L, V, Q, true><<<blocks, kZoThreads, 0, st>>>(
            rowptr, colind, vals, B, C, p->d_scratch, p->d_chunk_rows, p->d_chunk_starts,
            p->d_chunk_slot, p->num_chunks, N);
    } else {
        zo_chunk_kernel<L, V, Q, false><<<blocks, kZoThreads, 0, st>>>(
            rowptr, colind, vals, B, C, p->d_scratch, p->d_chunk_rows, p->d_chunk_starts,
            p->d_chunk_slot, p->num_chunks, N);
    }
}

// Launch sequence on caller-provided scratch (num_slots * N floats).
int zo_run_with_scratch(const RaZoPlan* p, float* scratch, const int* d_rowptr,
                        const int* d_colind, const float* d_vals, const float* d_B,
                        float* d_C, int N, cudaStream_t st, int phase_mask = 7)
{
    const bool wide_ok = (N % 4 == 0) && aligned16(d_B) && aligned16(d_C) &&
                         aligned16(scratch);
    const bool vec_a = aligned16(d_colind) && aligned16(d_vals);
    const int N4 = N / 4;
    RaZoPlan view = *p;            // shallow copy that carries the scratch pointer
    view.d_scratch = scratch;
    // RA_ZO_CHUNK_ENGINE=register runs the chunks on the register engine (diagnostic switch)
    // RA_ZO_CHUNK_ENGINE=register runs the chunks on the register engine (diagnostic switch)
    const char* engine_env = std::getenv("RA_ZO_CHUNK_ENGINE");
    const bool chunk_register = engine_env && std::string(engine_env) == "register";
    // A matrix made of long rows (nearly all work in chunks) at N >= 256 runs faster on the
    // register engine, as CSR_DIRECT does there: full chunks keep enough loads in flight and
    // every gathered byte crosses the shared-memory data path once.
    const bool long_rows = N >= 256 && (long long)p->num_chunks >= 16ll * p->num_small;
    const bool chunk_stream = wide_ok && stream_aligned_width_ok(N) && !chunk_register && !long_rows;
    if (p->num_chunks > 0 && p->num_small > 0 && (phase_mask & 3) == 3 && chunk_stream) {
        // chunks and small rows in one launch: the chunk warps (the long items) start first
        StreamArgs a{};
        a.rowptr = d_rowptr; a.colind = d_colind; a.vals = d_vals; a.B = d_B; a.C = d_C;
        a.scratch = scratch; a.chunk_rows = p->d_chunk_rows; a.chunk_starts = p->d_chunk_starts;
        a.chunk_slot = p->d_chunk_slot; a.num_chunks = p->num_chunks;
        a.row_ids = p->d_small_row_ids; a.num_items = p->num_small; a.N = N;
        const int rc = launch_csr_stream_aligned<kModeFused>(a, st);
        if (rc != RA_OK) return rc;
        phase_mask &= ~3;
    }
    if (p->num_chunks > 0 && (phase_mask & 1) && chunk_stream) {
        StreamArgs a{};
        a.rowptr = d_rowptr; a.colind = d_colind; a.vals = d_vals; a.B = d_B; a.C = d_C;
        a.scratch = scratch; a.chunk_rows = p->d_chunk_rows; a.chunk_starts = p->d_chunk_starts;
        a.chunk_slot = p->d_chunk_slot; a.num_items = p->num_chunks; a.N = N;
        const int rc = launch_csr_stream_aligned<kModeChunks>(a, st);
        if (rc != RA_OK) return rc;
    } else if (p->num_chunks > 0 && (phase_mask & 1)) {
        if (wide_ok && N4 == 8)        launch_chunks<8, 1, 4>(&view, d_rowptr, d_colind, d_vals, d_B, d_C, N, vec_a, st);
        else if (wide_ok && N4 == 16)  launch_chunks<16, 1, 2>(&view, d_rowptr, d_colind, d_vals, d_B, d_C, N, vec_a, st);
        else if (wide_ok && N4 == 32)  launch_chunks<32, 1, 1>(&view, d_rowptr, d_colind, d_vals, d_B, d_C, N, vec_a, st);
        else if (wide_ok && N4 == 64)  launch_chunks<32, 2, 1>(&view, d_rowptr, d_colind, d_vals, d_B, d_C, N, vec_a, st);
        else if (wide_ok && N4 == 128) launch_chunks<32, 4, 1>(&view, d_rowptr, d_colind, d_vals, d_B, d_C, N, vec_a, st);
        else {
            const int blocks = (int)(((i64)p->num_chunks * 32 + kZoThreads - 1) / kZoThreads);
            zo_chunk_generic_kernel<<<blocks, kZoThreads, 0, st>>>(
                d_rowptr, d_colind, d_vals, d_B, d_C, scratch, p->d_chunk_rows,
                p->d_chunk_starts, p->d_chunk_slot, p->num_chunks, N);
        }
        RA_KERNEL_CHECK();
    }
    if (p->num_small > 0 && (phase_mask & 2)) {
        const int rc = launch_csr_rows(d_rowptr, d_colind, d_vals, d_B, d_C,
                                       p->d_small_row_ids, p->num_small, N, st, -1);
        if (rc != RA_OK) return rc;
    }
    if (p->num_zero_rows > 0 && (phase_mask & 4)) {
        const int vec4 = (N % 4 == 0 && aligned16(d_C) && aligned16(scratch)) ? 1 : 0;
        const i64 threads = vec4 ? (i64)p->num_zero_rows * (N / 4) : (i64)p->num_zero_rows * 32;
        const int blocks = (int)std::max<i64>(1, std::min<i64>((threads + kZoThreads - 1) / kZoThreads, (i64)sm_count() * 32));
        zo_finish_kernel<<<blocks, kZoThreads, 0, st>>>(
            p->d_zero_row_ids, p->d_zero_slot_off, scratch, d_C, p->num_zero_rows, N, vec4);
        RA_KERNEL_CHECK();
    }
    return RA_OK;
}

}  // namespace ra

static int zo_run_common(RaZoPlan* p, const int32_t* d_rowptr, const int32_t* d_colind,
                         const float* d_vals, const float* d_B, float* d_C, int N,
                         int phase_mask, void* stream)
{
    using namespace ra;
    RA_REQUIRE(p != nullptr, RA_ERR_INVALID_ARG, "ra_zo_plan_run: plan is null");
    RA_REQUIRE(N >= 0, RA_ERR_INVALID_ARG, "ra_zo_plan_run: negative N");
    if (p->M == 0 || N == 0) return RA_OK;
    RA_REQUIRE(d_rowptr && d_C, RA_ERR_INVALID_ARG, "ra_zo_plan_run: null pointer");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const size_t need = (size_t)p->num_slots * (size_t)N * sizeof(float);
    if (need > p->scratch_bytes) {
        if (p->d_scratch) RA_CUDA_TRY(cudaFree(p->d_scratch));
        p->d_scratch = nullptr; p->scratch_bytes = 0;
        RA_CUDA_TRY(cudaMalloc(reinterpret_cast<void**>(&p->d_scratch), need));
        p->scratch_bytes = need;
    }
    return zo_run_with_scratch(p, p->d_scratch, d_rowptr, d_colind, d_vals, d_B, d_C, N, st,
                               phase_mask);
}

extern "C" int ra_zo_plan_run(RaZoPlan* p, const int32_t* d_rowptr, const int32_t* d_colind,
                              const float* d_vals, const float* d_B, float* d_C, int N,
                              void* stream)
{
    return zo_run_common(p, d_rowptr, d_colind, d_vals, d_B, d_C, N, 7, stream);
}

extern "C" int ra_zo_plan_run_phases(RaZoPlan* p, const int32_t* d_rowptr, const int32_t* d_colind,
                                     const float* d_vals, const float* d_B, float* d_C, int N,
                                     int phase_mask, void* stream)
{
    return zo_run_common(p, d_rowptr, d_colind, d_vals, d_B, d_C, N, phase_mask & 7, stream);
}

// ---------------------------------------------------------------------------
// Allocation-free run
//
// Some callers must not allocate device memory at run time: a serving loop that
// has handed every byte of HBM to its own pool, code running inside a region
// where cudaMalloc would synchronise the device (another stream is mid-flight),
// or a host that is simply not allowed to grow its footprint after start-up.
// ra_zo_plan_run grows the plan's scratch with cudaMalloc on first use; the
// entry point below never does. Its scratch is a fixed array that lives in the
// library image: every GPU that loads the library holds these 16 MiB until the
// process exits.
//
// The array's name below is a host-side handle, not a device address, so the
// address that the kernels receive is looked up with cudaGetSymbolAddress, once
// per device, with that device current.
// ---------------------------------------------------------------------------
namespace ra {
constexpr size_t kNoAllocScratchFloats = (size_t)4 << 20;       // 4 Mi floats = 16 MiB
static __device__ __align__(256) float g_zo_noalloc_scratch[kNoAllocScratchFloats];
static std::mutex g_noalloc_mutex;
static float* g_noalloc_ptr[64] = {};                            // per device ordinal
}  // namespace ra

extern "C" int ra_zo_plan_run_noalloc(RaZoPlan* p, const int32_t* d_rowptr, const int32_t* d_colind,
                                      const float* d_vals, const float* d_B, float* d_C, int N,
                                      void* stream)
{
    using namespace ra;
    RA_REQUIRE(p != nullptr, RA_ERR_INVALID_ARG, "ra_zo_plan_run_noalloc: plan is null");
    RA_REQUIRE(N >= 0, RA_ERR_INVALID_ARG, "ra_zo_plan_run_noalloc: negative N");
    if (p->M == 0 || N == 0) return RA_OK;
    RA_REQUIRE(d_rowptr && d_C, RA_ERR_INVALID_ARG, "ra_zo_plan_run_noalloc: null pointer");
    const size_t need = (size_t)p->num_slots * (size_t)N;
    RA_REQUIRE(need <= kNoAllocScratchFloats, RA_ERR_TOO_LARGE,
               "ra_zo_plan_run_noalloc: this plan needs %zu scratch floats (%d chunk slots x N=%d) but the "
               "built-in scratch holds %zu; use ra_zo_plan_run, which allocates",
               need, p->num_slots, N, kNoAllocScratchFloats);
    int dev = 0;
    RA_CUDA_TRY(cudaGetDevice(&dev));
    RA_REQUIRE(dev >= 0 && dev < 64, RA_ERR_UNSUPPORTED, "device ordinal %d out of range", dev);
    float* scratch = nullptr;
    {
        std::lock_guard<std::mutex> lock(g_noalloc_mutex);
        if (!g_noalloc_ptr[dev]) {
            void* addr = nullptr;
            RA_CUDA_TRY(cudaGetSymbolAddress(&addr, g_zo_noalloc_scratch));
            g_noalloc_ptr[dev] = static_cast<float*>(addr);
        }
        scratch = g_noalloc_ptr[dev];
    }
    return zo_run_with_scratch(p, scratch, d_rowptr, d_colind, d_vals, d_B, d_C, N,
                               static_cast<cudaStream_t>(stream));
}
