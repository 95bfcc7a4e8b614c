// Tile plan shared by the builder (tile_build.cu) and the kernels (tile_spmm.cu).
// Format (replaces RATcDirectPlan / RACommunityTCPlan / RASegmentHybridPlan,
// ra_common.h:593-719): rows are grouped in windows of 8; inside a window each
// distinct column is an 8x1 vector; 8 vectors form a block.
//   block_offsets[w]      first block of window w
//   atox[b*8 + k]         column (= B row) of vector k of block b, 0 for padding
//   vals_f16[b*64 + (r*4 + k/2)*2 + (k&1)]   fp16 value of (vector k, window row r)
//   val_masks/val_base/vals_zc   TC_DIRECT_ZC instead of vals_f16: bit k*8+r of val_masks[b]
//                         says (vector k, row r) is stored; its fp16 value is
//                         vals_zc[val_base[b] + popcount(mask bits below k*8+r)]
//   win_rows[w*8 + r]     COMMUNITY_TC: original row of window slot r, -1 = padding
//   seg_*/split_*         SEGMENT_HYBRID: <=64-block segments and merge tables
#pragma once

#include "common.cuh"

struct RaTilePlan {
    int kind = 0;
    int active = 0;
    int M = 0, K = 0;
    int num_windows = 0;
    long long num_blocks = 0;
    int max_window_blocks = 0;        // blocks of the largest window (engine choice at run time)
    long long nnz = 0;
    float tile_density = 0.f;
    int* d_block_offsets = nullptr;
    int* d_atox = nullptr;
    uint16_t* d_vals_f16 = nullptr;
    int* d_win_rows = nullptr;
    // TC_DIRECT_ZC (zero-compressed values; d_vals_f16 stays null)
    unsigned long long* d_val_masks = nullptr;
    int* d_val_base = nullptr;
    uint16_t* d_vals_zc = nullptr;
    // SEGMENT_HYBRID
    int num_segments = 0, num_split_segs = 0, num_split_windows = 0, num_zero_rows = 0;
    int* d_seg_window = nullptr;
    int* d_seg_bbegin = nullptr;
    int* d_seg_bend = nullptr;
    int* d_seg_scratch = nullptr;
    int* d_split_wins = nullptr;
    int* d_split_off = nullptr;
    int* d_zero_rows = nullptr;
    // lazily grown scratch (one plan must not run on two streams at once)
    uint16_t* d_bhalf = nullptr;      // fp16 copy of B for the FP16 path
    size_t bhalf_bytes = 0;
    float* d_scratch = nullptr;       // split-segment partial tiles
    size_t scratch_bytes = 0;
    int* d_status = nullptr;          // device status word of the kernels
};

namespace ra {
constexpr int kWindowRows   = 8;
constexpr int kVecPerBlock  = 8;
constexpr int kSegBlocks    = 64;
constexpr unsigned kSoleSegFlag = 0x80000000u;
}
