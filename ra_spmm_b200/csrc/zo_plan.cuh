// ZERO_OVERHEAD_CSR plan shared by the builder / kernels (zero_overhead.cu) and the plan
// file reader / writer (plan_io.cu). Replaces RAZeroOverheadPlan, ra_common.h:507-530.
#pragma once

#include "common.cuh"

struct RaZoPlan {
    int M = 0, K = 0;
    int num_tiny = 0, num_short = 0, num_medium = 0, num_long = 0, num_empty = 0;
    int num_small = 0, num_chunks = 0, num_zero_rows = 0, max_long_chunks = 0;
    int num_slots = 0;
    int* d_small_row_ids = nullptr;
    int* d_chunk_rows = nullptr;
    int* d_chunk_starts = nullptr;
    int* d_chunk_slot = nullptr;      // derived: scratch slot per chunk, -1 = sole
    int* d_zero_row_ids = nullptr;
    int* d_zero_slot_off = nullptr;   // derived: [num_zero_rows+1] slot ranges
    float* d_scratch = nullptr;       // lazily grown: num_slots * N floats
    size_t scratch_bytes = 0;
};
