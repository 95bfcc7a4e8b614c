// Plan files: a built ZERO_OVERHEAD_CSR or tile plan written to disk and read back.
//
// The reference keeps plans in memory only (RAZeroOverheadPlan / RATcDirectPlan /
// RACommunityTCPlan / RASegmentHybridPlan, ra_common.h:507-530, 593-719) and rebuilds them in
// every process; its experiments/verify_format_checksums.py expects per-array checksums of the
// formats to compare across runs. A plan file serves both: every array is stored with its
// length and its 64-bit FNV-1a checksum, the reader recomputes the checksums while it uploads,
// and a mismatch (truncated or edited file) is an error, not a silently different plan.
//
// File layout (little endian):
//   magic "RASPMMB2" | u32 version | u32 family (0 ZERO_OVERHEAD, 1 tile) | 16 x i64 scalars
//   then per array, in a fixed order per family: u64 bytes | u64 fnv1a64 | data, padded to 8 bytes
#include "tile_plan.cuh"
#include "zo_plan.cuh"

#include <cstring>
#include <memory>
#include <vector>

extern "C" int ra_zo_plan_destroy(RaZoPlan* p);
extern "C" int ra_tile_plan_destroy(RaTilePlan* p);

namespace ra {
namespace {

constexpr char kMagic[8] = {'R', 'A', 'S', 'P', 'M', 'M', 'B', '2'};
constexpr uint32_t kVersion = 1;
constexpr size_t kChunk = (size_t)32 << 20;           // staging buffer for device <-> file copies
constexpr int kScalars = 16;

struct File {
    FILE* f = nullptr;
    ~File() { if (f) std::fclose(f); }
};

inline uint64_t fnv_step(uint64_t h, const unsigned char* p, size_t n) {
    for (size_t i = 0; i < n; ++i) { h ^= p[i]; h *= 0x100000001b3ull; }
    return h;
}

// device array -> file, checksummed
int write_array(FILE* f, const void* d_ptr, size_t bytes, std::vector<unsigned char>& stage) {
    uint64_t head[2] = {(uint64_t)bytes, 0xcbf29ce484222325ull};
    const long head_pos = std::ftell(f);
    RA_REQUIRE(std::fwrite(head, sizeof(head), 1, f) == 1, RA_ERR_INVALID_ARG, "plan file: write failed");
    const unsigned char* src = static_cast<const unsigned char*>(d_ptr);
    for (size_t off = 0; off < bytes; off += kChunk) {
        const size_t n = std::min(kChunk, bytes - off);
        RA_CUDA_TRY(cudaMemcpy(stage.data(), src + off, n, cudaMemcpyDeviceToHost));
        head[1] = fnv_step(head[1], stage.data(), n);
        RA_REQUIRE(std::fwrite(stage.data(), 1, n, f) == n, RA_ERR_INVALID_ARG, "plan file: write failed");
    }
    const size_t pad = (8 - bytes % 8) % 8;
    const unsigned char zeros[8] = {0};
    if (pad) RA_REQUIRE(std::fwrite(zeros, 1, pad, f) == pad, RA_ERR_INVALID_ARG, "plan file: write failed");
    const long end_pos = std::ftell(f);
    std::fseek(f, head_pos, SEEK_SET);
    RA_REQUIRE(std::fwrite(head, sizeof(head), 1, f) == 1, RA_ERR_INVALID_ARG, "plan file: write failed");
    std::fseek(f, end_pos, SEEK_SET);
    return RA_OK;
}

// file -> freshly allocated device array; `expect_bytes` comes from the header scalars
int read_array(FILE* f, void** d_out, size_t expect_bytes, const char* name, std::vector<unsigned char>& stage) {
    uint64_t head[2];
    RA_REQUIRE(std::fread(head, sizeof(head), 1, f) == 1, RA_ERR_INVALID_ARG, "plan file: truncated before array %s", name);
    RA_REQUIRE(head[0] == expect_bytes, RA_ERR_INVALID_ARG,
               "plan file: array %s holds %llu bytes, the header implies %zu", name, (unsigned long long)head[0], expect_bytes);
    *d_out = nullptr;
    if (expect_bytes) RA_CUDA_TRY(cudaMalloc(d_out, expect_bytes));
    uint64_t h = 0xcbf29ce484222325ull;
    unsigned char* dst = static_cast<unsigned char*>(*d_out);
    for (size_t off = 0; off < expect_bytes; off += kChunk) {
        const size_t n = std::min(kChunk, expect_bytes - off);
        RA_REQUIRE(std::fread(stage.data(), 1, n, f) == n, RA_ERR_INVALID_ARG, "plan file: truncated inside array %s", name);
        h = fnv_step(h, stage.data(), n);
        RA_CUDA_TRY(cudaMemcpy(dst + off, stage.data(), n, cudaMemcpyHostToDevice));
    }
    RA_REQUIRE(h == head[1], RA_ERR_INVALID_ARG,
               "plan file: checksum of array %s is %016llx, the file says %016llx", name,
               (unsigned long long)h, (unsigned long long)head[1]);
    const size_t pad = (8 - expect_bytes % 8) % 8;
    if (pad) std::fseek(f, (long)pad, SEEK_CUR);
    return RA_OK;
}

int write_header(FILE* f, uint32_t family, const int64_t (&sc)[kScalars]) {
    RA_REQUIRE(std::fwrite(kMagic, 8, 1, f) == 1 && std::fwrite(&kVersion, 4, 1, f) == 1 &&
               std::fwrite(&family, 4, 1, f) == 1 && std::fwrite(sc, sizeof(sc), 1, f) == 1,
               RA_ERR_INVALID_ARG, "plan file: write failed");
    return RA_OK;
}

int read_header(FILE* f, uint32_t family, int64_t (&sc)[kScalars]) {
    char magic[8]; uint32_t version = 0, fam = 0;
    RA_REQUIRE(std::fread(magic, 8, 1, f) == 1 && std::fread(&version, 4, 1, f) == 1 &&
               std::fread(&fam, 4, 1, f) == 1 && std::fread(sc, sizeof(sc), 1, f) == 1,
               RA_ERR_INVALID_ARG, "plan file: truncated header");
    RA_REQUIRE(std::memcmp(magic, kMagic, 8) == 0, RA_ERR_INVALID_ARG, "plan file: not a plan file (bad magic)");
    RA_REQUIRE(version == kVersion, RA_ERR_UNSUPPORTED, "plan file: version %u, this library reads %u", version, kVersion);
    RA_REQUIRE(fam == family, RA_ERR_INVALID_ARG, "plan file: holds a %s plan, a %s plan was asked for",
               fam == 0 ? "ZERO_OVERHEAD_CSR" : "tile", family == 0 ? "ZERO_OVERHEAD_CSR" : "tile");
    for (int i = 0; i < kScalars; ++i)
        RA_REQUIRE(sc[i] >= 0 && sc[i] < ((int64_t)1 << 40), RA_ERR_INVALID_ARG, "plan file: header field %d out of range", i);
    return RA_OK;
}

}  // namespace
}  // namespace ra

extern "C" int ra_zo_plan_save(const RaZoPlan* p, const char* path)
{
    using namespace ra;
    RA_REQUIRE(p && path, RA_ERR_INVALID_ARG, "ra_zo_plan_save: null argument");
    File file; file.f = std::fopen(path, "wb");
    RA_REQUIRE(file.f, RA_ERR_INVALID_ARG, "ra_zo_plan_save: cannot open %s for writing", path);
    const int64_t sc[kScalars] = {p->M, p->K, p->num_tiny, p->num_short, p->num_medium, p->num_long, p->num_empty,
                                  p->num_small, p->num_chunks, p->num_zero_rows, p->max_long_chunks, p->num_slots};
    int rc = write_header(file.f, 0, sc);
    std::vector<unsigned char> stage(kChunk);
    const struct { const void* ptr; size_t n; } arrays[] = {
        {p->d_small_row_ids, (size_t)p->num_small}, {p->d_chunk_rows, (size_t)p->num_chunks},
        {p->d_chunk_starts, (size_t)p->num_chunks}, {p->d_chunk_slot, (size_t)p->num_chunks},
        {p->d_zero_row_ids, (size_t)p->num_zero_rows},
        {p->d_zero_slot_off, p->M > 0 ? (size_t)p->num_zero_rows + 1 : 0}};
    RA_CUDA_TRY(cudaDeviceSynchronize());
    for (const auto& a : arrays) {
        if (rc != RA_OK) break;
        rc = write_array(file.f, a.ptr, a.n * sizeof(int), stage);
    }
    return rc;
}

extern "C" int ra_zo_plan_load(const char* path, RaZoPlan** out)
{
    using namespace ra;
    RA_REQUIRE(path && out, RA_ERR_INVALID_ARG, "ra_zo_plan_load: null argument");
    *out = nullptr;
    File file; file.f = std::fopen(path, "rb");
    RA_REQUIRE(file.f, RA_ERR_INVALID_ARG, "ra_zo_plan_load: cannot open %s", path);
    int64_t sc[kScalars];
    int rc = read_header(file.f, 0, sc);
    if (rc != RA_OK) return rc;
    RaZoPlan* p = new RaZoPlan();
    p->M = (int)sc[0]; p->K = (int)sc[1]; p->num_tiny = (int)sc[2]; p->num_short = (int)sc[3];
    p->num_medium = (int)sc[4]; p->num_long = (int)sc[5]; p->num_empty = (int)sc[6]; p->num_small = (int)sc[7];
    p->num_chunks = (int)sc[8]; p->num_zero_rows = (int)sc[9]; p->max_long_chunks = (int)sc[10]; p->num_slots = (int)sc[11];
    std::vector<unsigned char> stage(kChunk);
    const struct { int** ptr; size_t n; const char* name; } arrays[] = {
        {&p->d_small_row_ids, (size_t)p->num_small, "small_row_ids"}, {&p->d_chunk_rows, (size_t)p->num_chunks, "chunk_rows"},
        {&p->d_chunk_starts, (size_t)p->num_chunks, "chunk_starts"}, {&p->d_chunk_slot, (size_t)p->num_chunks, "chunk_slot"},
        {&p->d_zero_row_ids, (size_t)p->num_zero_rows, "zero_row_ids"},
        {&p->d_zero_slot_off, p->M > 0 ? (size_t)p->num_zero_rows + 1 : 0, "zero_slot_off"}};
    for (const auto& a : arrays) {
        rc = read_array(file.f, reinterpret_cast<void**>(a.ptr), a.n * sizeof(int), a.name, stage);
        if (rc != RA_OK) { ra_zo_plan_destroy(p); return rc; }
    }
    *out = p;
    return RA_OK;
}

namespace ra {
namespace {
// array table of a tile plan: pointer slot, element size, element count from the plan's scalars
struct TileArray { void** slot; size_t elem; size_t count; const char* name; };

std::vector<TileArray> tile_arrays(RaTilePlan* p)
{
    std::vector<TileArray> v;
    if (!p->active) return v;
    const size_t nb = (size_t)p->num_blocks, W = (size_t)p->num_windows;
    v.push_back({reinterpret_cast<void**>(&p->d_block_offsets), 4, W + 1, "block_offsets"});
    v.push_back({reinterpret_cast<void**>(&p->d_atox), 4, 8 * nb, "atox"});
    if (p->kind == RA_TILE_TC_DIRECT_ZC) {
        v.push_back({reinterpret_cast<void**>(&p->d_val_masks), 8, nb, "val_masks"});
        v.push_back({reinterpret_cast<void**>(&p->d_val_base), 4, nb, "val_base"});
        v.push_back({reinterpret_cast<void**>(&p->d_vals_zc), 2, (size_t)p->nnz, "vals_zc"});
    } else {
        v.push_back({reinterpret_cast<void**>(&p->d_vals_f16), 2, 64 * nb, "vals_f16"});
    }
    if (p->kind == RA_TILE_COMMUNITY_TC)
        v.push_back({reinterpret_cast<void**>(&p->d_win_rows), 4, 8 * W, "win_rows"});
    if (p->kind == RA_TILE_SEGMENT_HYBRID) {
        const size_t S = (size_t)p->num_segments, Q = (size_t)p->num_split_windows;
        v.push_back({reinterpret_cast<void**>(&p->d_seg_window), 4, S, "seg_window"});
        v.push_back({reinterpret_cast<void**>(&p->d_seg_bbegin), 4, S, "seg_bbegin"});
        v.push_back({reinterpret_cast<void**>(&p->d_seg_bend), 4, S, "seg_bend"});
        v.push_back({reinterpret_cast<void**>(&p->d_seg_scratch), 4, S, "seg_scratch"});
        v.push_back({reinterpret_cast<void**>(&p->d_split_wins), 4, Q, "split_wins"});
        v.push_back({reinterpret_cast<void**>(&p->d_split_off), 4, Q + 1, "split_off"});
        v.push_back({reinterpret_cast<void**>(&p->d_zero_rows), 4, (size_t)p->num_zero_rows, "zero_rows"});
    }
    return v;
}
}  // namespace
}  // namespace ra

extern "C" int ra_tile_plan_save(const RaTilePlan* plan, const char* path)
{
    using namespace ra;
    RA_REQUIRE(plan && path, RA_ERR_INVALID_ARG, "ra_tile_plan_save: null argument");
    RaTilePlan* p = const_cast<RaTilePlan*>(plan);          // the table takes pointer slots; nothing is written
    File file; file.f = std::fopen(path, "wb");
    RA_REQUIRE(file.f, RA_ERR_INVALID_ARG, "ra_tile_plan_save: cannot open %s for writing", path);
    int32_t density_bits; std::memcpy(&density_bits, &p->tile_density, 4);
    const int64_t sc[kScalars] = {p->kind, p->active, p->M, p->K, p->num_windows, p->num_blocks, p->nnz,
                                  (int64_t)(uint32_t)density_bits, p->num_segments, p->num_split_segs,
                                  p->num_split_windows, p->num_zero_rows, p->max_window_blocks};
    int rc = write_header(file.f, 1, sc);
    std::vector<unsigned char> stage(kChunk);
    RA_CUDA_TRY(cudaDeviceSynchronize());
    for (const auto& a : tile_arrays(p)) {
        if (rc != RA_OK) break;
        rc = write_array(file.f, *a.slot, a.elem * a.count, stage);
    }
    return rc;
}

extern "C" int ra_tile_plan_load(const char* path, RaTilePlan** out)
{
    using namespace ra;
    RA_REQUIRE(path && out, RA_ERR_INVALID_ARG, "ra_tile_plan_load: null argument");
    *out = nullptr;
    File file; file.f = std::fopen(path, "rb");
    RA_REQUIRE(file.f, RA_ERR_INVALID_ARG, "ra_tile_plan_load: cannot open %s", path);
    int64_t sc[kScalars];
    int rc = read_header(file.f, 1, sc);
    if (rc != RA_OK) return rc;
    RA_REQUIRE(sc[0] <= RA_TILE_TC_DIRECT_ZC, RA_ERR_INVALID_ARG, "plan file: unknown tile plan kind %lld", (long long)sc[0]);
    RaTilePlan* p = new RaTilePlan();
    p->kind = (int)sc[0]; p->active = (int)sc[1]; p->M = (int)sc[2]; p->K = (int)sc[3];
    p->num_windows = (int)sc[4]; p->num_blocks = sc[5]; p->nnz = sc[6];
    const int32_t density_bits = (int32_t)(uint32_t)sc[7]; std::memcpy(&p->tile_density, &density_bits, 4);
    p->num_segments = (int)sc[8]; p->num_split_segs = (int)sc[9]; p->num_split_windows = (int)sc[10];
    p->num_zero_rows = (int)sc[11]; p->max_window_blocks = (int)sc[12];
    std::vector<unsigned char> stage(kChunk);
    for (const auto& a : tile_arrays(p)) {
        rc = read_array(file.f, a.slot, a.elem * a.count, a.name, stage);
        if (rc != RA_OK) { ra_tile_plan_destroy(p); return rc; }
    }
    if (p->active) {
        cudaError_t e = cudaMalloc(reinterpret_cast<void**>(&p->d_status), sizeof(int));
        if (e == cudaSuccess) e = cudaMemset(p->d_status, 0, sizeof(int));
        if (e != cudaSuccess) {
            set_error("ra_tile_plan_load: %s", cudaGetErrorString(e));
            ra_tile_plan_destroy(p);
            return RA_ERR_CUDA;
        }
    }
    *out = p;
    return RA_OK;
}
