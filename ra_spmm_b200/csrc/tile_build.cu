// Tile-format plan builders on the device, bit-exact with the reference's host
// builders: build_ra_tc_direct_plan_impl (tc/ra_tc_direct.cu:627-780),
// make_ra_community_tc_plan (tc/ra_community_tc.cu:320-471) and
// make_ra_segment_hybrid_plan (tc/ra_segment_hybrid.cu:371-543).
//
// The reference sorts, per window, the (column, window row, value) entries and
// numbers the distinct columns; here one stable radix sort orders every entry
// of the matrix by (window, column, row slot) - the window is the top key
// field, so windows stay contiguous - and a prefix sum over "first entry of a
// (window, column) pair" flags numbers the vectors. The COMMUNITY_TC row order
// (rows sorted by first stored column, ties by row id, empty rows last) is a
// stable radix sort of the rows by that column.
//
// Precondition shared with the reference: no duplicate (row, column) pairs.
// Columns inside a row may be in any order.
#include "radix_sort.cuh"
#include "tile_plan.cuh"

#include <climits>
#include <vector>

namespace ra {

constexpr int kTbThreads = 256;

static int bits_for(unsigned long long max_value) {   // bits needed to store max_value
    int b = 1;
    while (b < 64 && (max_value >> b) != 0ull) ++b;
    return b;
}

// key = first stored column of the row (INT_MAX when empty), payload = row
__global__ void __launch_bounds__(kTbThreads)
tb_row_keys_kernel(const int* __restrict__ rowptr, const int* __restrict__ colind, int M,
                   unsigned long long* __restrict__ keys, unsigned* __restrict__ payload)
{
    for (i64 r = (i64)blockIdx.x * blockDim.x + threadIdx.x; r < M; r += (i64)gridDim.x * blockDim.x) {
        const int s = rowptr[r], e = rowptr[r + 1];
        keys[r] = (unsigned long long)(unsigned)((s < e) ? colind[s] : INT_MAX);
        payload[r] = (unsigned)r;
    }
}

// win_rows[i] = order[i] (padding -1); pos[order[i]] = i
__global__ void __launch_bounds__(kTbThreads)
tb_win_rows_kernel(const unsigned* __restrict__ order, int M, int padded,
                   int* __restrict__ win_rows, int* __restrict__ pos)
{
    for (i64 i = (i64)blockIdx.x * blockDim.x + threadIdx.x; i < padded; i += (i64)gridDim.x * blockDim.x) {
        if (i < M) {
            const int r = (int)order[i];
            win_rows[i] = r;
            pos[r] = (int)i;
        } else {
            win_rows[i] = -1;
        }
    }
}

// One warp per row: key = window << shift_w | col << 3 | slot, payload = nnz index
__global__ void __launch_bounds__(kTbThreads)
tb_entry_keys_kernel(const int* __restrict__ rowptr, const int* __restrict__ colind,
                     const int* __restrict__ pos, int M, int shift_w,
                     unsigned long long* __restrict__ keys, unsigned* __restrict__ payload)
{
    const int lane = threadIdx.x & 31;
    const i64 warps = ((i64)gridDim.x * blockDim.x) >> 5;
    for (i64 r = ((i64)blockIdx.x * blockDim.x + threadIdx.x) >> 5; r < M; r += warps) {
        const int s = rowptr[r], e = rowptr[r + 1];
        const unsigned long long P = (unsigned long long)(pos ? pos[r] : (int)r);
        const unsigned long long hi = ((P >> 3) << shift_w) | (P & 7ull);
        for (int p = s + lane; p < e; p += 32) {
            keys[p] = hi | ((unsigned long long)(unsigned)colind[p] << 3);
            payload[p] = (unsigned)p;
        }
    }
}

__global__ void __launch_bounds__(kTbThreads)
tb_heads_kernel(const unsigned long long* __restrict__ keys, i64 n, int* __restrict__ heads)
{
    for (i64 i = (i64)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (i64)gridDim.x * blockDim.x) {
        heads[i] = (i == 0 || (keys[i] >> 3) != (keys[i - 1] >> 3)) ? 1 : 0;
    }
}

// ws[w] = first sorted entry of window w (w in [0, W]); blocks[w] from the head scan
__global__ void __launch_bounds__(kTbThreads)
tb_window_bounds_kernel(const unsigned long long* __restrict__ keys, i64 n, int W, int shift_w,
                        int* __restrict__ ws)
{
    for (i64 w = (i64)blockIdx.x * blockDim.x + threadIdx.x; w <= W; w += (i64)gridDim.x * blockDim.x) {
        const unsigned long long target = (unsigned long long)w << shift_w;
        i64 lo = 0, hi = n;
        while (lo < hi) {
            const i64 mid = (lo + hi) >> 1;
            if (keys[mid] < target) lo = mid + 1; else hi = mid;
        }
        ws[w] = (int)lo;
    }
}

__global__ void __launch_bounds__(kTbThreads)
tb_window_blocks_kernel(const int* __restrict__ ws, const int* __restrict__ hscan, int W,
                        int* __restrict__ blocks, int* __restrict__ max_blocks)
{
    int local_max = 0;
    for (i64 w = (i64)blockIdx.x * blockDim.x + threadIdx.x; w < W; w += (i64)gridDim.x * blockDim.x) {
        const int nvec = hscan[ws[w + 1]] - hscan[ws[w]];
        const int nb = (nvec + kVecPerBlock - 1) / kVecPerBlock;
        blocks[w] = nb;
        local_max = max(local_max, nb);
    }
    if (local_max > 0) atomicMax(max_blocks, local_max);
}

// fp32 -> fp16 bits, round to nearest even. The reference converts on the host with two
// routines that differ for NaN only: TC_DIRECT (padded and zero-compressed plans) maps every
// value whose exponent field is all ones - NaN included - to the infinity of its sign
// (host_float_to_half_bits, tc/ra_tc_direct.cu:45-69); COMMUNITY_TC and SEGMENT_HYBRID keep
// the canonical NaN of __float2half_rn (tc/ra_community_tc.cu:35-38, tc/ra_segment_hybrid.cu:34-37).
__device__ __forceinline__ uint16_t tb_half_bits(float v, int nan_to_inf)
{
    if (nan_to_inf && v != v) return (uint16_t)(((__float_as_uint(v) >> 16) & 0x8000u) | 0x7C00u);
    return __half_as_ushort(__float2half_rn(v));
}

__global__ void __launch_bounds__(kTbThreads)
tb_fill_kernel(const unsigned long long* __restrict__ keys, const unsigned* __restrict__ payload,
               const float* __restrict__ vals, const int* __restrict__ hscan,
               const int* __restrict__ ws, const int* __restrict__ block_offsets, i64 n,
               int shift_w, unsigned long long col_mask, int* __restrict__ atox,
               uint16_t* __restrict__ vals_f16, int nan_to_inf)
{
    for (i64 i = (i64)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (i64)gridDim.x * blockDim.x) {
        const unsigned long long key = keys[i];
        const int w = (int)(key >> shift_w);
        const int col = (int)((key >> 3) & col_mask);
        const int slot = (int)(key & 7ull);
        const int h0 = hscan[i], h1 = hscan[i + 1];
        const int v = h1 - 1 - hscan[ws[w]];              // vector slot inside the window
        const i64 b = (i64)block_offsets[w] + (v >> 3);
        const int k = v & 7;
        if (h1 != h0) atox[b * kVecPerBlock + k] = col;
        vals_f16[b * 64 + (slot * 4 + (k >> 1)) * 2 + (k & 1)] = tb_half_bits(vals[payload[i]], nan_to_inf);
    }
}

// Zero-compressed values (tc/ra_tc_direct.cu:686-735): sorted entry i is stored value i;
// a block's mask collects the (vector, row) bits of its entries and its base is the index of
// its first entry (entries of a window start at rowptr[8w], as in the reference).
__global__ void __launch_bounds__(kTbThreads)
tb_fill_zc_kernel(const unsigned long long* __restrict__ keys, const unsigned* __restrict__ payload,
                  const float* __restrict__ vals, const int* __restrict__ hscan,
                  const int* __restrict__ ws, const int* __restrict__ block_offsets, i64 n,
                  int shift_w, unsigned long long col_mask, int* __restrict__ atox,
                  unsigned long long* __restrict__ val_masks, int* __restrict__ val_base,
                  uint16_t* __restrict__ vals_zc)
{
    for (i64 i = (i64)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (i64)gridDim.x * blockDim.x) {
        const unsigned long long key = keys[i];
        const int w = (int)(key >> shift_w);
        const int col = (int)((key >> 3) & col_mask);
        const int slot = (int)(key & 7ull);
        const int h0 = hscan[i], h1 = hscan[i + 1];
        const int v = h1 - 1 - hscan[ws[w]];
        const i64 b = (i64)block_offsets[w] + (v >> 3);
        const int k = v & 7;
        if (h1 != h0) {
            atox[b * kVecPerBlock + k] = col;
            if (k == 0) val_base[b] = (int)i;            // first entry of the block
        }
        atomicOr(val_masks + b, 1ull << (k * 8 + slot));
        vals_zc[i] = tb_half_bits(vals[payload[i]], 1);
    }
}

// ---- SEGMENT_HYBRID split tables --------------------------------------------
// per window: segments, split flag, scratch slots, rows to list
__global__ void __launch_bounds__(kTbThreads)
sg_count_kernel(const int* __restrict__ block_offsets, int W, int M, int* __restrict__ cnt, i64 stride)
{
    for (i64 w = (i64)blockIdx.x * blockDim.x + threadIdx.x; w < W; w += (i64)gridDim.x * blockDim.x) {
        const int nblk = block_offsets[w + 1] - block_offsets[w];
        const bool split = nblk > kSegBlocks;
        const int nseg = split ? (nblk + kSegBlocks - 1) / kSegBlocks : 1;
        const int rows = min(M, (int)(w + 1) * kWindowRows) - (int)w * kWindowRows;
        cnt[0 * stride + w] = nseg;
        cnt[1 * stride + w] = split ? 1 : 0;
        cnt[2 * stride + w] = split ? nseg : 0;
        cnt[3 * stride + w] = split ? rows : 0;
    }
}

__global__ void __launch_bounds__(kTbThreads)
sg_fill_kernel(const int* __restrict__ block_offsets, int W, int M, const int* __restrict__ off,
               i64 stride, int total_slots, int num_split,
               int* __restrict__ seg_window, int* __restrict__ seg_bbegin,
               int* __restrict__ seg_bend, int* __restrict__ seg_scratch,
               int* __restrict__ split_wins, int* __restrict__ split_off, int* __restrict__ zero_rows)
{
    for (i64 w = (i64)blockIdx.x * blockDim.x + threadIdx.x; w < W; w += (i64)gridDim.x * blockDim.x) {
        const int b0 = block_offsets[w], b1 = block_offsets[w + 1];
        const int s0 = off[0 * stride + w];
        if (b1 - b0 <= kSegBlocks) {
            seg_window[s0] = (int)((unsigned)w | kSoleSegFlag);
            seg_bbegin[s0] = b0;
            seg_bend[s0] = b1;
            seg_scratch[s0] = -1;
        } else {
            const int q = off[1 * stride + w];
            const int slot0 = off[2 * stride + w];
            split_wins[q] = (int)w;
            split_off[q] = slot0;
            int j = 0;
            for (int b = b0; b < b1; b += kSegBlocks, ++j) {
                seg_window[s0 + j] = (int)w;
                seg_bbegin[s0 + j] = b;
                seg_bend[s0 + j] = min(b + kSegBlocks, b1);
                seg_scratch[s0 + j] = slot0 + j;
            }
            const int z0 = off[3 * stride + w];
            const int rows = min(M, (int)(w + 1) * kWindowRows) - (int)w * kWindowRows;
            for (int r = 0; r < rows; ++r) zero_rows[z0 + r] = (int)w * kWindowRows + r;
        }
    }
    if (blockIdx.x == 0 && threadIdx.x == 0) split_off[num_split] = total_slots;
}

struct DevMem {   // owning temporary
    void* p = nullptr;
    ~DevMem() { if (p) cudaFree(p); }
    template <typename T> T* as() { return static_cast<T*>(p); }
};

static int grid_for(i64 work, int threads = kTbThreads) {
    i64 g = (work + threads - 1) / threads;
    const i64 cap = (i64)sm_count() * 16;
    if (g > cap) g = cap;
    if (g < 1) g = 1;
    return (int)g;
}

}  // namespace ra

extern "C" int ra_tile_plan_destroy(RaTilePlan* p)
{
    if (!p) return RA_OK;
    cudaFree(p->d_block_offsets); cudaFree(p->d_atox); cudaFree(p->d_vals_f16);
    cudaFree(p->d_win_rows);
    cudaFree(p->d_val_masks); cudaFree(p->d_val_base); cudaFree(p->d_vals_zc);
    cudaFree(p->d_seg_window); cudaFree(p->d_seg_bbegin); cudaFree(p->d_seg_bend);
    cudaFree(p->d_seg_scratch); cudaFree(p->d_split_wins); cudaFree(p->d_split_off);
    cudaFree(p->d_zero_rows);
    cudaFree(p->d_bhalf); cudaFree(p->d_scratch); cudaFree(p->d_status);
    delete p;
    return RA_OK;
}

extern "C" int ra_tile_plan_create(int kind, const int32_t* rowptr, const int32_t* colind,
                                   const float* vals, int csr_on_device,
                                   int M, int K, int N, void* stream, RaTilePlan** out)
{
    using namespace ra;
    RA_REQUIRE(out != nullptr, RA_ERR_INVALID_ARG, "ra_tile_plan_create: out is null");
    *out = nullptr;
    RA_REQUIRE(kind >= RA_TILE_TC_DIRECT && kind <= RA_TILE_TC_DIRECT_ZC, RA_ERR_INVALID_ARG,
               "ra_tile_plan_create: unknown kind %d", kind);
    cudaStream_t st = static_cast<cudaStream_t>(stream);

    RaTilePlan* p = new RaTilePlan();
    p->kind = kind; p->M = M; p->K = K;
    auto fail = [&](int code) { ra_tile_plan_destroy(p); return code; };
#define TB_TRY(expr) do { cudaError_t _e = (expr); if (_e != cudaSuccess) { \
        ra::set_error("%s failed at %s:%d: %s", #expr, __FILE__, __LINE__, cudaGetErrorString(_e)); \
        return fail(RA_ERR_CUDA); } } while (0)

    // inactive plans: same conditions as the reference builders
    if (M <= 0 || K <= 0 || N < 16 || rowptr == nullptr) { *out = p; return RA_OK; }

    DevMem rp_d, ci_d, va_d;
    const int* d_rowptr = rowptr; const int* d_colind = colind; const float* d_vals = vals;
    int nnz = 0;
    if (csr_on_device) {
        TB_TRY(cudaMemcpyAsync(&nnz, rowptr + M, sizeof(int), cudaMemcpyDeviceToHost, st));
        TB_TRY(cudaStreamSynchronize(st));
    } else {
        nnz = rowptr[M];
    }
    if (nnz <= 0) { *out = p; return RA_OK; }
    if (colind == nullptr || vals == nullptr) {
        set_error("ra_tile_plan_create: colind/vals are null");
        return fail(RA_ERR_INVALID_ARG);
    }
    if (!csr_on_device) {
        TB_TRY(cudaMalloc(&rp_d.p, sizeof(int) * ((size_t)M + 1)));
        TB_TRY(cudaMalloc(&ci_d.p, sizeof(int) * (size_t)nnz));
        TB_TRY(cudaMalloc(&va_d.p, sizeof(float) * (size_t)nnz));
        TB_TRY(cudaMemcpyAsync(rp_d.p, rowptr, sizeof(int) * ((size_t)M + 1), cudaMemcpyHostToDevice, st));
        TB_TRY(cudaMemcpyAsync(ci_d.p, colind, sizeof(int) * (size_t)nnz, cudaMemcpyHostToDevice, st));
        TB_TRY(cudaMemcpyAsync(va_d.p, vals, sizeof(float) * (size_t)nnz, cudaMemcpyHostToDevice, st));
        d_rowptr = rp_d.as<int>(); d_colind = ci_d.as<int>(); d_vals = va_d.as<float>();
    }

    const int W = (M + kWindowRows - 1) / kWindowRows;
    const i64 n = nnz;
    const i64 nsort = std::max<i64>(n, M);
    DevMem k0, k1, v0, v1, tmp, hs, wsb, blk, pos_d;
    TB_TRY(cudaMalloc(&k0.p, sizeof(unsigned long long) * (size_t)nsort));
    TB_TRY(cudaMalloc(&k1.p, sizeof(unsigned long long) * (size_t)nsort));
    TB_TRY(cudaMalloc(&v0.p, sizeof(unsigned) * (size_t)nsort));
    TB_TRY(cudaMalloc(&v1.p, sizeof(unsigned) * (size_t)nsort));
    TB_TRY(cudaMalloc(&tmp.p, sizeof(int) * (size_t)std::max(rs_tmp_ints(nsort), scan_tmp_ints(nsort + 1))));
    TB_TRY(cudaMalloc(&hs.p, sizeof(int) * ((size_t)n + 1)));
    TB_TRY(cudaMalloc(&wsb.p, sizeof(int) * ((size_t)W + 1)));
    TB_TRY(cudaMalloc(&blk.p, sizeof(int) * ((size_t)W + 1)));

    // ---- COMMUNITY_TC: locality order --------------------------------------
    const int* d_pos = nullptr;
    if (kind == RA_TILE_COMMUNITY_TC) {
        TB_TRY(cudaMalloc(&pos_d.p, sizeof(int) * (size_t)M));
        TB_TRY(cudaMalloc(reinterpret_cast<void**>(&p->d_win_rows), sizeof(int) * (size_t)W * kWindowRows));
        tb_row_keys_kernel<<<grid_for(M), kTbThreads, 0, st>>>(d_rowptr, d_colind, M,
                                                               k0.as<unsigned long long>(), v0.as<unsigned>());
        TB_TRY(cudaGetLastError());
        bool in_first = true;
        TB_TRY(radix_sort_pairs(k0.as<unsigned long long>(), v0.as<unsigned>(),
                                k1.as<unsigned long long>(), v1.as<unsigned>(), M, 32,
                                tmp.as<int>(), st, &in_first));
        const unsigned* order = in_first ? v0.as<unsigned>() : v1.as<unsigned>();
        tb_win_rows_kernel<<<grid_for((i64)W * kWindowRows), kTbThreads, 0, st>>>(
            order, M, W * kWindowRows, p->d_win_rows, pos_d.as<int>());
        TB_TRY(cudaGetLastError());
        d_pos = pos_d.as<int>();
    }

    // ---- sort all entries by (window, column, row slot) ----------------------
    const int col_bits = bits_for((unsigned long long)(K > 0 ? K - 1 : 0));
    const int shift_w = col_bits + 3;
    const int w_bits = bits_for((unsigned long long)(W > 0 ? W - 1 : 0));
    const int key_bits = shift_w + w_bits;
    {
        const i64 warps_needed = M;
        const int g = grid_for(warps_needed * 32);
        tb_entry_keys_kernel<<<g, kTbThreads, 0, st>>>(d_rowptr, d_colind, d_pos, M, shift_w,
                                                       k0.as<unsigned long long>(), v0.as<unsigned>());
        TB_TRY(cudaGetLastError());
    }
    bool in_first = true;
    TB_TRY(radix_sort_pairs(k0.as<unsigned long long>(), v0.as<unsigned>(),
                            k1.as<unsigned long long>(), v1.as<unsigned>(), n, key_bits,
                            tmp.as<int>(), st, &in_first));
    const unsigned long long* skeys = in_first ? k0.as<unsigned long long>() : k1.as<unsigned long long>();
    const unsigned* spay = in_first ? v0.as<unsigned>() : v1.as<unsigned>();

    // ---- number the vectors, size the windows --------------------------------
    tb_heads_kernel<<<grid_for(n), kTbThreads, 0, st>>>(skeys, n, hs.as<int>());
    TB_TRY(cudaGetLastError());
    TB_TRY(exclusive_scan_i32(hs.as<int>(), hs.as<int>(), n, tmp.as<int>(), st));
    tb_window_bounds_kernel<<<grid_for((i64)W + 1), kTbThreads, 0, st>>>(skeys, n, W, shift_w, wsb.as<int>());
    TB_TRY(cudaGetLastError());
    TB_TRY(cudaMalloc(reinterpret_cast<void**>(&p->d_status), sizeof(int)));     // doubles as the max-reduction cell here
    TB_TRY(cudaMemsetAsync(p->d_status, 0, sizeof(int), st));
    tb_window_blocks_kernel<<<grid_for(W), kTbThreads, 0, st>>>(wsb.as<int>(), hs.as<int>(), W, blk.as<int>(), p->d_status);
    TB_TRY(cudaGetLastError());
    TB_TRY(cudaMalloc(reinterpret_cast<void**>(&p->d_block_offsets), sizeof(int) * ((size_t)W + 1)));
    TB_TRY(exclusive_scan_i32(blk.as<int>(), p->d_block_offsets, W, tmp.as<int>(), st));
    int total_blocks = 0, total_vectors = 0;
    TB_TRY(cudaMemcpyAsync(&total_blocks, p->d_block_offsets + W, sizeof(int), cudaMemcpyDeviceToHost, st));
    TB_TRY(cudaMemcpyAsync(&total_vectors, hs.as<int>() + n, sizeof(int), cudaMemcpyDeviceToHost, st));
    TB_TRY(cudaMemcpyAsync(&p->max_window_blocks, p->d_status, sizeof(int), cudaMemcpyDeviceToHost, st));
    TB_TRY(cudaStreamSynchronize(st));

    // ---- fill atox / vals_f16 ------------------------------------------------
    const size_t atox_bytes = sizeof(int) * (size_t)total_blocks * kVecPerBlock;
    const size_t vals_bytes = sizeof(uint16_t) * (size_t)total_blocks * 64;
    TB_TRY(cudaMalloc(reinterpret_cast<void**>(&p->d_atox), atox_bytes));
    TB_TRY(cudaMemsetAsync(p->d_atox, 0, atox_bytes, st));
    const unsigned long long col_mask = (1ull << col_bits) - 1ull;
    if (kind == RA_TILE_TC_DIRECT_ZC) {
        const size_t mask_bytes = sizeof(unsigned long long) * (size_t)total_blocks;
        TB_TRY(cudaMalloc(reinterpret_cast<void**>(&p->d_val_masks), mask_bytes));
        TB_TRY(cudaMalloc(reinterpret_cast<void**>(&p->d_val_base), sizeof(int) * (size_t)total_blocks));
        TB_TRY(cudaMalloc(reinterpret_cast<void**>(&p->d_vals_zc), sizeof(uint16_t) * (size_t)n));
        TB_TRY(cudaMemsetAsync(p->d_val_masks, 0, mask_bytes, st));
        tb_fill_zc_kernel<<<grid_for(n), kTbThreads, 0, st>>>(skeys, spay, d_vals, hs.as<int>(), wsb.as<int>(),
                                                             p->d_block_offsets, n, shift_w, col_mask,
                                                             p->d_atox, p->d_val_masks, p->d_val_base,
                                                             p->d_vals_zc);
    } else {
        TB_TRY(cudaMalloc(reinterpret_cast<void**>(&p->d_vals_f16), vals_bytes));
        TB_TRY(cudaMemsetAsync(p->d_vals_f16, 0, vals_bytes, st));
        tb_fill_kernel<<<grid_for(n), kTbThreads, 0, st>>>(skeys, spay, d_vals, hs.as<int>(), wsb.as<int>(),
                                                          p->d_block_offsets, n, shift_w, col_mask,
                                                          p->d_atox, p->d_vals_f16,
                                                          kind == RA_TILE_TC_DIRECT ? 1 : 0);
    }
    TB_TRY(cudaGetLastError());

    p->num_windows = W;
    p->num_blocks = total_blocks;
    p->nnz = n;
    p->tile_density = (total_blocks > 0)
        ? static_cast<float>(static_cast<double>(n) /
                             (static_cast<double>((i64)total_blocks * kVecPerBlock) * kWindowRows))
        : 0.f;
    (void)total_vectors;

    // ---- SEGMENT_HYBRID: balance split -----------------------------------------
    if (kind == RA_TILE_SEGMENT_HYBRID) {
        DevMem cnt;
        const i64 stride = (i64)W + 1;
        TB_TRY(cudaMalloc(&cnt.p, sizeof(int) * (size_t)(4 * stride)));
        sg_count_kernel<<<grid_for(W), kTbThreads, 0, st>>>(p->d_block_offsets, W, M, cnt.as<int>(), stride);
        TB_TRY(cudaGetLastError());
        int totals[4];
        for (int c = 0; c < 4; ++c) {
            TB_TRY(exclusive_scan_i32(cnt.as<int>() + c * stride, cnt.as<int>() + c * stride, W,
                                      tmp.as<int>(), st));
            TB_TRY(cudaMemcpyAsync(&totals[c], cnt.as<int>() + c * stride + W, sizeof(int),
                                   cudaMemcpyDeviceToHost, st));
        }
        TB_TRY(cudaStreamSynchronize(st));
        p->num_segments = totals[0];
        p->num_split_windows = totals[1];
        p->num_split_segs = totals[2];
        p->num_zero_rows = totals[3];
        auto alloc_ints = [&](int** ptr, size_t cnt_ints) -> cudaError_t {
            return cudaMalloc(reinterpret_cast<void**>(ptr), sizeof(int) * std::max<size_t>(cnt_ints, 1));
        };
        TB_TRY(alloc_ints(&p->d_seg_window, (size_t)p->num_segments));
        TB_TRY(alloc_ints(&p->d_seg_bbegin, (size_t)p->num_segments));
        TB_TRY(alloc_ints(&p->d_seg_bend, (size_t)p->num_segments));
        TB_TRY(alloc_ints(&p->d_seg_scratch, (size_t)p->num_segments));
        TB_TRY(alloc_ints(&p->d_split_wins, (size_t)p->num_split_windows));
        TB_TRY(alloc_ints(&p->d_split_off, (size_t)p->num_split_windows + 1));
        TB_TRY(alloc_ints(&p->d_zero_rows, (size_t)p->num_zero_rows));
        sg_fill_kernel<<<grid_for(W), kTbThreads, 0, st>>>(
            p->d_block_offsets, W, M, cnt.as<int>(), stride, p->num_split_segs, p->num_split_windows,
            p->d_seg_window, p->d_seg_bbegin, p->d_seg_bend, p->d_seg_scratch, p->d_split_wins,
            p->d_split_off, p->d_zero_rows);
        TB_TRY(cudaGetLastError());
        TB_TRY(cudaStreamSynchronize(st));
    }
    TB_TRY(cudaMemsetAsync(p->d_status, 0, sizeof(int), st));         // allocated above (held the window maximum)
    TB_TRY(cudaStreamSynchronize(st));   // temporaries are freed on return
#undef TB_TRY
    p->active = 1;
    *out = p;
    return RA_OK;
}

extern "C" int ra_tile_plan_device_status(RaTilePlan* p, int* status)
{
    using namespace ra;
    RA_REQUIRE(p && status, RA_ERR_INVALID_ARG, "ra_tile_plan_device_status: null argument");
    *status = 0;
    if (!p->d_status) return RA_OK;
    RA_CUDA_TRY(cudaDeviceSynchronize());
    RA_CUDA_TRY(cudaMemcpy(status, p->d_status, sizeof(int), cudaMemcpyDeviceToHost));
    if (*status != 0) RA_CUDA_TRY(cudaMemset(p->d_status, 0, sizeof(int)));   // read and clear
    return RA_OK;
}

extern "C" int ra_tile_plan_info(const RaTilePlan* p, RaTileInfo* o)
{
    using namespace ra;
    RA_REQUIRE(p && o, RA_ERR_INVALID_ARG, "ra_tile_plan_info: null argument");
    *o = RaTileInfo{};
    o->kind = p->kind; o->active = p->active; o->M = p->M; o->K = p->K;
    o->num_windows = p->num_windows; o->num_blocks = p->num_blocks; o->nnz = p->nnz;
    o->tile_density = p->tile_density;
    // accounting of the reference builders (tc/ra_tc_direct.cu:767-776,
    // tc/ra_community_tc.cu:465-468, tc/ra_segment_hybrid.cu:535-539)
    int64_t bytes = 0;
    if (p->active) {
        bytes = (int64_t)sizeof(int) * (p->num_windows + 1) + (int64_t)sizeof(int) * p->num_blocks * 8;
        if (p->kind == RA_TILE_TC_DIRECT_ZC)
            bytes += (int64_t)(sizeof(unsigned long long) + sizeof(int)) * p->num_blocks +
                     (int64_t)sizeof(uint16_t) * p->nnz;
        else
            bytes += (int64_t)sizeof(uint16_t) * p->num_blocks * 64;
        if (p->kind == RA_TILE_COMMUNITY_TC) bytes += (int64_t)sizeof(int) * p->num_windows * 8;
        if (p->kind == RA_TILE_SEGMENT_HYBRID)
            bytes += (int64_t)sizeof(int) * (3LL * p->num_segments + p->num_zero_rows);
    }
    o->plan_bytes = bytes;
    o->d_block_offsets = p->d_block_offsets; o->d_atox = p->d_atox; o->d_vals_f16 = p->d_vals_f16;
    o->d_win_rows = p->d_win_rows;
    o->num_segments = p->num_segments; o->num_split_segs = p->num_split_segs;
    o->num_split_windows = p->num_split_windows; o->num_zero_rows = p->num_zero_rows;
    o->d_seg_window = p->d_seg_window; o->d_seg_bbegin = p->d_seg_bbegin; o->d_seg_bend = p->d_seg_bend;
    o->d_seg_scratch = p->d_seg_scratch; o->d_split_wins = p->d_split_wins;
    o->d_split_off = p->d_split_off; o->d_zero_rows = p->d_zero_rows;
    o->d_val_masks = reinterpret_cast<const uint64_t*>(p->d_val_masks);
    o->d_val_base = p->d_val_base; o->d_vals_zc = p->d_vals_zc;
    return RA_OK;
}
