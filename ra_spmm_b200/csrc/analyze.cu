// Structural analysis of a CSR matrix: the 34 features that compute_router_features
// (router/router_features.cpp:113-432) extracts for the research portfolio and that the
// binding analyze_matrix publishes (bindings/ra_bindings.cpp:1993-2051).
//
// The reference walks the matrix on one host thread and counts the nonempty 16x16 tiles in a
// hash map. Here everything that is O(nnz) runs on the device and yields integers only, so it
// is exact whatever the order of evaluation:
//   * one warp per row: first / last stored column, the sum of the columns (u64) and the
//     64-bucket column signature; the same pass emits the tile key of every entry;
//   * the tile keys are radix-sorted; run lengths give a histogram "tiles with c entries",
//     c = 1..256, which determines every tile statistic (the reference sorts the fills before it
//     reduces them, so the histogram carries the same information as its sorted vector);
//   * the proxy row order (centroid bucket, column span, longer rows first, stable) is two
//     chained stable radix sorts of the rows.
// The floating-point reductions whose result depends on the order of the additions (variance
// of the degrees and of the fills, means over windows) then run on the host over M-sized
// arrays in the reference's order, which keeps every field bit-exact.
#include "radix_sort.cuh"

#include <algorithm>
#include <cmath>
#include <cstring>
#include <vector>

namespace ra {
namespace {

constexpr int kAnTile = 16;          // tile edge of the fill statistics
constexpr int kAnSigBuckets = 64;    // column buckets of a row signature
constexpr int kAnWindow = 16;        // rows per window of the partition proxies
constexpr int kAnThreads = 256;
constexpr int kAnMaxTileCount = kAnTile * kAnTile;
constexpr float kAnCandidateFill = 0.25f;   // TC_FILL_THRESHOLD, ra_common.h:762

struct AnMem {   // owning device temporary
    void* p = nullptr;
    ~AnMem() { if (p) cudaFree(p); }
    template <typename T> T* as() const { return static_cast<T*>(p); }
};

// One warp per row: proxies of the row and the tile key of each of its entries.
__global__ void __launch_bounds__(kAnThreads)
an_rows_kernel(const int* __restrict__ rowptr, const int* __restrict__ colind, int M, int K, i64 tile_cols,
               int* __restrict__ first_col, int* __restrict__ last_col,
               unsigned long long* __restrict__ col_sum, unsigned long long* __restrict__ signature,
               unsigned long long* __restrict__ tile_key)
{
    const int lane = threadIdx.x & 31;
    const i64 warp0 = ((i64)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const i64 warps = ((i64)gridDim.x * blockDim.x) >> 5;
    const i64 kdiv = K > 1 ? K : 1;
    for (i64 r = warp0; r < M; r += warps) {
        const int b = __ldg(rowptr + r), e = __ldg(rowptr + r + 1);
        unsigned long long sum = 0ull, sig = 0ull;
        const i64 trow = (r / kAnTile) * tile_cols;
        for (int p = b + lane; p < e; p += 32) {
            const int c = ld_stream_int(colind + p);
            sum += (unsigned long long)(unsigned)c;
            i64 bucket = ((i64)c * kAnSigBuckets) / kdiv;
            bucket = bucket < kAnSigBuckets - 1 ? bucket : kAnSigBuckets - 1;
            sig |= 1ull << (int)(bucket < 0 ? 0 : bucket);
            tile_key[p] = (unsigned long long)(trow + c / kAnTile);
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            sum += __shfl_xor_sync(0xffffffffu, sum, o);
            sig |= __shfl_xor_sync(0xffffffffu, sig, o);
        }
        if (lane == 0) {
            first_col[r] = e > b ? __ldg(colind + b) : 0;
            last_col[r] = e > b ? __ldg(colind + e - 1) : 0;
            col_sum[r] = sum;
            signature[r] = sig;
        }
    }
}

// Sorted tile keys -> hist[c] = number of tiles with c entries (c = 1..256); hist[257] counts
// runs longer than a tile can hold.
__global__ void __launch_bounds__(kAnThreads)
an_tile_hist_kernel(const unsigned long long* __restrict__ keys, i64 n, unsigned long long* __restrict__ hist)
{
    __shared__ unsigned int sh[kAnMaxTileCount + 2];
    for (int i = threadIdx.x; i < kAnMaxTileCount + 2; i += blockDim.x) sh[i] = 0u;
    __syncthreads();
    const i64 stride = (i64)gridDim.x * blockDim.x;
    for (i64 i = (i64)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
        const unsigned long long k = keys[i];
        if (i + 1 < n && keys[i + 1] == k) continue;          // not the last entry of its tile
        int count = 1;
        while (count <= kAnMaxTileCount && i - count >= 0 && keys[i - count] == k) ++count;
        atomicAdd(&sh[count <= kAnMaxTileCount ? count : kAnMaxTileCount + 1], 1u);
    }
    __syncthreads();
    for (int i = threadIdx.x; i < kAnMaxTileCount + 2; i += blockDim.x)
        if (sh[i]) atomicAdd(hist + i, (unsigned long long)sh[i]);
}

// Centroid of a row exactly as the host computes it: float(double(sum) / double(len)).
__device__ __forceinline__ float an_centroid(unsigned long long sum, int len) {
    return len > 0 ? __double2float_rn(__ddiv_rn((double)sum, (double)len)) : 0.f;
}

// Keys of the proxy row order. pass 0: longer rows first; pass 1 (on the rows in the order
// pass 0 left them): centroid bucket, then column span.
__global__ void __launch_bounds__(kAnThreads)
an_order_keys_kernel(int pass, const unsigned* __restrict__ rows_in, const int* __restrict__ rowptr,
                     const int* __restrict__ first_col, const int* __restrict__ last_col,
                     const unsigned long long* __restrict__ col_sum, int M, int K,
                     unsigned long long* __restrict__ key, unsigned* __restrict__ rows_out)
{
    const i64 i = (i64)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= M) return;
    const unsigned r = pass == 0 ? (unsigned)i : rows_in[i];
    const int len = __ldg(rowptr + r + 1) - __ldg(rowptr + r);
    if (pass == 0) {
        key[i] = (unsigned long long)(0x7fffffff - len);
        rows_out[i] = r;
        return;
    }
    int bucket = 0;
    if (K > 0) bucket = (int)__fdiv_rn(__fmul_rn(an_centroid(col_sum[r], len), 16.f), (float)K);
    bucket = bucket < 0 ? 0 : (bucket > 31 ? 31 : bucket);
    const int span = len > 0 ? (last_col[r] - first_col[r] + 1) : K;
    key[i] = ((unsigned long long)bucket << 32) | (unsigned long long)((unsigned)span ^ 0x80000000u);
}

inline float an_clamp01(float x) { return std::max(0.f, std::min(1.f, x)); }
inline float an_div(float num, float den) { return (std::fabs(den) > 1e-6f) ? (num / den) : 0.f; }
inline float an_jaccard(unsigned long long a, unsigned long long b) {
    const int uni = __builtin_popcountll(a | b);
    return uni == 0 ? 0.f : (float)__builtin_popcountll(a & b) / (float)uni;
}

// mean of a sequence of floats accumulated in double in sequence order
struct AnMean {
    double sum = 0.0;
    size_t n = 0;
    void add(float v) { sum += (double)v; ++n; }
    float value() const { return n == 0 ? 0.f : (float)(sum / (double)n); }
};

}  // namespace
}  // namespace ra

extern "C" int ra_analyze_matrix(const int32_t* rowptr, const int32_t* colind, int on_device,
                                 int M, int K, int N, void* stream, RaMatrixAnalysis* out)
{
    using namespace ra;
    RA_REQUIRE(out != nullptr, RA_ERR_INVALID_ARG, "ra_analyze_matrix: out is null");
    std::memset(out, 0, sizeof(*out));
    if (M <= 0 || K <= 0) return RA_OK;                       // the reference returns zeros
    RA_REQUIRE(rowptr != nullptr, RA_ERR_INVALID_ARG, "ra_analyze_matrix: rowptr is null");
    cudaStream_t st = static_cast<cudaStream_t>(stream);

    // ---- rowptr on the host, both arrays on the device ----
    std::vector<int> rp((size_t)M + 1);
    AnMem rp_d, ci_d;
    const int* d_rowptr = rowptr; const int* d_colind = colind;
    if (on_device) {
        RA_CUDA_TRY(cudaMemcpyAsync(rp.data(), rowptr, sizeof(int) * rp.size(), cudaMemcpyDeviceToHost, st));
        RA_CUDA_TRY(cudaStreamSynchronize(st));
    } else {
        std::memcpy(rp.data(), rowptr, sizeof(int) * rp.size());
    }
    const int nnz = rp[M];
    out->matrix_M = M; out->matrix_K = K; out->output_dim_N = N; out->total_nnz = nnz;
    if (nnz <= 0) return RA_OK;
    RA_REQUIRE(colind != nullptr, RA_ERR_INVALID_ARG, "ra_analyze_matrix: colind is null");
    if (!on_device) {
        RA_CUDA_TRY(cudaMalloc(&rp_d.p, sizeof(int) * rp.size()));
        RA_CUDA_TRY(cudaMalloc(&ci_d.p, sizeof(int) * (size_t)nnz));
        RA_CUDA_TRY(cudaMemcpyAsync(rp_d.p, rowptr, sizeof(int) * rp.size(), cudaMemcpyHostToDevice, st));
        RA_CUDA_TRY(cudaMemcpyAsync(ci_d.p, colind, sizeof(int) * (size_t)nnz, cudaMemcpyHostToDevice, st));
        d_rowptr = rp_d.as<int>(); d_colind = ci_d.as<int>();
    }

    // ---- device pass 1: row proxies + tile keys ----
    const i64 tile_rows = ((i64)M + kAnTile - 1) / kAnTile;
    const i64 tile_cols = ((i64)K + kAnTile - 1) / kAnTile;
    const i64 nsort = std::max<i64>(nnz, M);
    AnMem first_d, last_d, sum_d, sig_d, k0, k1, v0, v1, tmp, hist_d;
    RA_CUDA_TRY(cudaMalloc(&first_d.p, sizeof(int) * (size_t)M));
    RA_CUDA_TRY(cudaMalloc(&last_d.p, sizeof(int) * (size_t)M));
    RA_CUDA_TRY(cudaMalloc(&sum_d.p, sizeof(unsigned long long) * (size_t)M));
    RA_CUDA_TRY(cudaMalloc(&sig_d.p, sizeof(unsigned long long) * (size_t)M));
    RA_CUDA_TRY(cudaMalloc(&k0.p, sizeof(unsigned long long) * (size_t)nsort));
    RA_CUDA_TRY(cudaMalloc(&k1.p, sizeof(unsigned long long) * (size_t)nsort));
    RA_CUDA_TRY(cudaMalloc(&v0.p, sizeof(unsigned) * (size_t)nsort));
    RA_CUDA_TRY(cudaMalloc(&v1.p, sizeof(unsigned) * (size_t)nsort));
    RA_CUDA_TRY(cudaMalloc(&tmp.p, sizeof(int) * (size_t)rs_tmp_ints(nsort)));
    RA_CUDA_TRY(cudaMalloc(&hist_d.p, sizeof(unsigned long long) * (kAnMaxTileCount + 2)));
    RA_CUDA_TRY(cudaMemsetAsync(hist_d.p, 0, sizeof(unsigned long long) * (kAnMaxTileCount + 2), st));
    RA_CUDA_TRY(cudaMemsetAsync(v0.p, 0, sizeof(unsigned) * (size_t)nsort, st));   // payload of the tile sort is unused

    const int grid_rows = (int)std::min<i64>(((i64)M * 32 + kAnThreads - 1) / kAnThreads, (i64)sm_count() * 16);
    an_rows_kernel<<<grid_rows, kAnThreads, 0, st>>>(d_rowptr, d_colind, M, K, tile_cols, first_d.as<int>(),
                                                     last_d.as<int>(), sum_d.as<unsigned long long>(),
                                                     sig_d.as<unsigned long long>(), k0.as<unsigned long long>());
    RA_KERNEL_CHECK();

    // ---- device pass 2: tiles with c entries ----
    int key_bits = 1;
    while (key_bits < 64 && ((unsigned long long)(tile_rows * tile_cols - 1) >> key_bits) != 0ull) ++key_bits;
    bool in_first = true;
    RA_CUDA_TRY(radix_sort_pairs(k0.as<unsigned long long>(), v0.as<unsigned>(), k1.as<unsigned long long>(),
                                 v1.as<unsigned>(), nnz, key_bits, tmp.as<int>(), st, &in_first));
    const int grid_hist = (int)std::min<i64>(((i64)nnz + kAnThreads - 1) / kAnThreads, (i64)sm_count() * 8);
    an_tile_hist_kernel<<<grid_hist, kAnThreads, 0, st>>>(in_first ? k0.as<unsigned long long>() : k1.as<unsigned long long>(),
                                                          nnz, hist_d.as<unsigned long long>());
    RA_KERNEL_CHECK();

    // ---- device pass 3: proxy row order = stable sort by (bucket, span) of the rows sorted by length ----
    const int grid_m = (int)(((i64)M + kAnThreads - 1) / kAnThreads);
    an_order_keys_kernel<<<grid_m, kAnThreads, 0, st>>>(0, nullptr, d_rowptr, first_d.as<int>(), last_d.as<int>(),
                                                        sum_d.as<unsigned long long>(), M, K,
                                                        k0.as<unsigned long long>(), v0.as<unsigned>());
    RA_KERNEL_CHECK();
    RA_CUDA_TRY(radix_sort_pairs(k0.as<unsigned long long>(), v0.as<unsigned>(), k1.as<unsigned long long>(),
                                 v1.as<unsigned>(), M, 31, tmp.as<int>(), st, &in_first));
    unsigned* rows_sorted = in_first ? v0.as<unsigned>() : v1.as<unsigned>();
    unsigned long long* key_a = in_first ? k0.as<unsigned long long>() : k1.as<unsigned long long>();
    unsigned long long* key_b = in_first ? k1.as<unsigned long long>() : k0.as<unsigned long long>();
    unsigned* rows_b = in_first ? v1.as<unsigned>() : v0.as<unsigned>();
    an_order_keys_kernel<<<grid_m, kAnThreads, 0, st>>>(1, rows_sorted, d_rowptr, first_d.as<int>(), last_d.as<int>(),
                                                        sum_d.as<unsigned long long>(), M, K, key_a, nullptr);
    RA_KERNEL_CHECK();
    bool in_a = true;
    RA_CUDA_TRY(radix_sort_pairs(key_a, rows_sorted, key_b, rows_b, M, 37, tmp.as<int>(), st, &in_a));
    const unsigned* order_d = in_a ? rows_sorted : rows_b;

    // ---- results to the host ----
    std::vector<int> first((size_t)M), last((size_t)M);
    std::vector<unsigned long long> col_sum((size_t)M), sig((size_t)M);
    std::vector<unsigned> order((size_t)M);
    unsigned long long hist[kAnMaxTileCount + 2];
    RA_CUDA_TRY(cudaMemcpyAsync(first.data(), first_d.p, sizeof(int) * (size_t)M, cudaMemcpyDeviceToHost, st));
    RA_CUDA_TRY(cudaMemcpyAsync(last.data(), last_d.p, sizeof(int) * (size_t)M, cudaMemcpyDeviceToHost, st));
    RA_CUDA_TRY(cudaMemcpyAsync(col_sum.data(), sum_d.p, sizeof(unsigned long long) * (size_t)M, cudaMemcpyDeviceToHost, st));
    RA_CUDA_TRY(cudaMemcpyAsync(sig.data(), sig_d.p, sizeof(unsigned long long) * (size_t)M, cudaMemcpyDeviceToHost, st));
    RA_CUDA_TRY(cudaMemcpyAsync(order.data(), order_d, sizeof(unsigned) * (size_t)M, cudaMemcpyDeviceToHost, st));
    RA_CUDA_TRY(cudaMemcpyAsync(hist, hist_d.p, sizeof(hist), cudaMemcpyDeviceToHost, st));
    RA_CUDA_TRY(cudaStreamSynchronize(st));
    RA_REQUIRE(hist[kAnMaxTileCount + 1] == 0ull, RA_ERR_UNSUPPORTED,
               "ra_analyze_matrix: a 16x16 tile holds more than 256 entries (duplicate (row, column) pairs)");

    RaMatrixAnalysis& f = *out;

    // ---- degree statistics (router_features.cpp:139-202) ----
    double sum_lens = 0.0;
    int max_len = 0;
    int top[5] = {-1, -1, -1, -1, -1};                        // five longest rows, descending
    for (int r = 0; r < M; ++r) {
        const int len = rp[r + 1] - rp[r];
        sum_lens += (double)len;
        max_len = std::max(max_len, len);
        if (len > top[4]) {
            int j = 4;
            while (j > 0 && top[j - 1] < len) { top[j] = top[j - 1]; --j; }
            top[j] = len;
        }
    }
    const double avg = sum_lens / (double)M;
    double var = 0.0;
    int dense_rows = 0, long_rows = 0;
    long long long_row_nnz = 0;
    const double long_row_threshold = std::max(32.0, 2.0 * avg);
    for (int r = 0; r < M; ++r) {
        const int len = rp[r + 1] - rp[r];
        const double delta = (double)len - avg;
        var += delta * delta;
        if (len > 2.0 * avg) ++dense_rows;
        if ((double)len >= long_row_threshold) { ++long_rows; long_row_nnz += len; }
    }
    const double std_dev = std::sqrt(var / (double)std::max(1, M));
    long long top5_nnz = 0;
    for (int i = 0; i < std::min(5, M); ++i) top5_nnz += top[i];
    f.avg_nnz_per_row = (float)avg;
    f.std_nnz_per_row = (float)std_dev;
    f.degree_cv = (avg > 1e-6) ? (float)(std_dev / avg) : 0.f;
    f.max_to_mean_ratio = (avg > 1e-6) ? (float)((double)max_len / avg) : 0.f;
    f.frac_dense_rows = (float)dense_rows / (float)std::max(1, M);
    f.skew_ratio = f.max_to_mean_ratio;
    f.long_row_fraction = (float)long_rows / (float)std::max(1, M);
    f.long_row_nnz_fraction = (float)long_row_nnz / (float)std::max(1, nnz);
    f.top_1_row_nnz_fraction = (float)(long long)top[0] / (float)std::max(1, nnz);
    f.top_5_row_nnz_fraction = (float)top5_nnz / (float)std::max(1, nnz);

    // ---- tile statistics from the histogram (router_features.cpp:204-258) ----
    // The reference's sorted fill vector holds hist[c] copies of c/256 for c = 1..256 in turn.
    unsigned long long tiles = 0, candidate_tiles = 0;
    long long candidate_nnz = 0;
    double fill_sum = 0.0;                                    // exact: multiples of 1/256
    for (int c = 1; c <= kAnMaxTileCount; ++c) {
        const float fill = (float)c / (float)kAnMaxTileCount;
        tiles += hist[c];
        fill_sum += (double)fill * (double)hist[c];
        if (fill >= kAnCandidateFill) { candidate_tiles += hist[c]; candidate_nnz += (long long)c * (long long)hist[c]; }
    }
    auto fill_at = [&](unsigned long long index) {            // element `index` of the sorted fills
        unsigned long long seen = 0;
        for (int c = 1; c <= kAnMaxTileCount; ++c) {
            seen += hist[c];
            if (index < seen) return (float)c / (float)kAnMaxTileCount;
        }
        return 0.f;
    };
    const float fill_mean = tiles == 0 ? 0.f : (float)(fill_sum / (double)tiles);
    double fill_var = 0.0;
    for (int c = 1; c <= kAnMaxTileCount; ++c) {
        const double delta = (double)((float)c / (float)kAnMaxTileCount) - (double)fill_mean;
        const double sq = delta * delta;
        for (unsigned long long i = 0; i < hist[c]; ++i) fill_var += sq;   // one addition per tile, as the reference adds them
    }
    fill_var = tiles == 0 ? 0.0 : fill_var / (double)tiles;
    f.tile_fill_mean = fill_mean;
    f.tile_fill_median = tiles == 0 ? 0.f : fill_at(tiles / 2);
    f.tile_fill_p90 = tiles == 0 ? 0.f : fill_at(std::min(tiles - 1, (tiles * 9) / 10));
    f.tile_fill_max = tiles == 0 ? 0.f : fill_at(tiles - 1);
    f.tile_fill_variance = (float)fill_var;
    f.tile_occupancy = (float)tiles / (float)std::max<long long>(1, tile_rows * tile_cols);
    f.actual_nnz_coverage = (float)candidate_nnz / (float)std::max(1, nnz);
    f.avg_nnz_per_tile = tiles == 0 ? 0.f : (float)nnz / (float)tiles;
    f.tc_candidate_tiles = (int)candidate_tiles;
    f.tc_candidate_ratio = tiles == 0 ? 0.f : (float)f.tc_candidate_tiles / (float)tiles;

    // ---- row similarity in stored order and in the proxy order (router_features.cpp:260-303) ----
    auto len_of = [&](unsigned r) { return rp[r + 1] - rp[r]; };
    AnMean adjacent, reordered;
    for (int r = 1; r < M; ++r) {
        if (len_of(r - 1) == 0 || len_of(r) == 0) continue;
        adjacent.add(an_jaccard(sig[r - 1], sig[r]));
    }
    f.local_row_similarity_proxy = adjacent.value();
    for (int i = 1; i < M; ++i) {
        const unsigned a = order[i - 1], b = order[i];
        if (len_of(a) == 0 || len_of(b) == 0) continue;
        reordered.add(an_jaccard(sig[a], sig[b]));
    }
    f.reordered_locality_proxy = reordered.value();

    // ---- 16-row windows (router_features.cpp:305-388) ----
    AnMean compactness_mean, similarity_mean, irregular_mean;
    long long tc_window_nnz = 0, cuda_window_nnz = 0;
    int irregular_windows = 0;
    for (int base = 0; base < M; base += kAnWindow) {
        const int end = std::min(M, base + kAnWindow);
        long long window_nnz = 0, long_window_nnz = 0;
        int min_col = K, max_col = -1, max_row_len = 0, sim_count = 0;
        float sim_sum = 0.f;
        for (int r = base; r < end; ++r) {
            const int len = len_of(r);
            window_nnz += len;
            max_row_len = std::max(max_row_len, len);
            if (len > 0) { min_col = std::min(min_col, first[r]); max_col = std::max(max_col, last[r]); }
            if (r > base && len_of(r - 1) > 0 && len > 0) { sim_sum += an_jaccard(sig[r - 1], sig[r]); ++sim_count; }
        }
        const float avg_row_len = (float)window_nnz / (float)std::max(1, end - base);
        const float window_long_threshold = std::max(32.f, 2.5f * avg_row_len);
        for (int r = base; r < end; ++r)
            if ((float)len_of(r) >= window_long_threshold) long_window_nnz += len_of(r);
        const int span = (max_col >= min_col) ? (max_col - min_col + 1) : K;
        const float compactness = (float)window_nnz / (float)std::max(1, (end - base) * std::max(1, span));
        const float similarity = (sim_count > 0) ? (sim_sum / (float)sim_count) : 0.f;
        const int aligned_span = std::max(16, ((span + 15) / 16) * 16);
        const float tile_density = (float)window_nnz / (float)std::max(16, (end - base) * aligned_span);
        const float compactness_norm = an_clamp01(compactness * 6.f);
        const float density_norm = an_clamp01(tile_density * 10.f);
        const float uniformity_norm = an_clamp01(1.f - an_div((float)max_row_len, 4.f * avg_row_len + 1.f));
        const float long_mass = an_div((float)long_window_nnz, (float)std::max<long long>(1, window_nnz));
        compactness_mean.add(compactness);
        similarity_mean.add(similarity);
        const float tc_score = 0.35f * compactness_norm + 0.30f * similarity + 0.20f * density_norm + 0.15f * uniformity_norm;
        const float irregular_score = 0.40f * long_mass +
                                      0.25f * an_clamp01(an_div((float)max_row_len, avg_row_len + 1.f) / 6.f) +
                                      0.20f * (1.f - compactness_norm) + 0.15f * (1.f - similarity);
        irregular_mean.add(irregular_score);
        if (avg_row_len >= 8.f && tc_score >= 0.55f && irregular_score < 0.45f) tc_window_nnz += window_nnz;
        if (irregular_score >= 0.50f || long_mass >= 0.20f) { cuda_window_nnz += window_nnz; ++irregular_windows; }
    }

    // ---- derived proxies (router_features.cpp:390-430) ----
    f.row_window_colspan_compactness = compactness_mean.value();
    const float window_similarity_mean = similarity_mean.value();
    const float window_irregular_mean = irregular_mean.value();
    f.tc_synergy_proxy = 0.35f * an_clamp01(f.tile_fill_mean / 0.20f) + 0.25f * f.tc_candidate_ratio +
                         0.20f * f.reordered_locality_proxy + 0.20f * f.row_window_colspan_compactness;
    f.locality_gain_proxy = an_clamp01(f.reordered_locality_proxy - f.local_row_similarity_proxy);
    const float ordered_locality = an_clamp01(f.local_row_similarity_proxy * an_clamp01(f.row_window_colspan_compactness * 2.f));
    f.locality_selectivity_proxy = an_clamp01(f.locality_gain_proxy * (1.f - ordered_locality));
    f.road_likeness_proxy = an_clamp01(f.local_row_similarity_proxy * an_clamp01(1.f - f.degree_cv / 0.35f) *
                                       an_clamp01(1.f - f.avg_nnz_per_row / 24.f) *
                                       an_clamp01(f.row_window_colspan_compactness / 0.25f));
    const float skew_branch = 0.45f * an_clamp01((f.skew_ratio - 2.0f) / 6.0f) + 0.30f * f.long_row_nnz_fraction +
                              0.15f * an_clamp01(f.top_1_row_nnz_fraction / 0.0020f) +
                              0.10f * an_clamp01(f.top_5_row_nnz_fraction / 0.0100f);
    const float n_scale = an_clamp01(((float)N - 128.f) / 384.f);
    const float dense_regular_branch = an_clamp01(f.avg_nnz_per_row / 192.f) * (0.35f + 0.65f * n_scale);
    f.row_split_affinity_proxy = an_clamp01(std::max(skew_branch, dense_regular_branch));
    f.estimated_tc_partition_ratio = an_clamp01((float)tc_window_nnz / (float)std::max(1, nnz));
    f.estimated_cuda_partition_ratio = an_clamp01((float)cuda_window_nnz / (float)std::max(1, nnz));
    f.irregular_window_fraction = (float)irregular_windows / (float)std::max(1, (M + kAnWindow - 1) / kAnWindow);
    const float partition_balance =
        an_div(2.f * std::min(f.estimated_tc_partition_ratio, f.estimated_cuda_partition_ratio),
               f.estimated_tc_partition_ratio + f.estimated_cuda_partition_ratio + 1e-6f);
    f.mixedness_proxy = an_clamp01(partition_balance *
                                   an_clamp01((f.estimated_tc_partition_ratio + f.estimated_cuda_partition_ratio) / 0.60f));
    f.tc_granularity_proxy = 0.55f * an_clamp01(f.avg_nnz_per_row / 64.f) +
                             0.45f * an_clamp01((1.f - f.long_row_fraction) + 0.5f * f.locality_selectivity_proxy);
    f.redundancy_risk_proxy = an_clamp01(0.45f * f.long_row_nnz_fraction + 0.30f * (1.f - f.row_window_colspan_compactness) +
                                         0.15f * (1.f - window_similarity_mean) + 0.10f * window_irregular_mean);
    return RA_OK;
}
