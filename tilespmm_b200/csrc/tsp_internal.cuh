// Internal declarations shared by the translation units of libtilespmm_b200.so.
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include <string>
#include <vector>

#include "../../include/tilespmm_b200.h"

// ---------------------------------------------------------------- errors

void tsp_set_error(const char *fmt, ...);

#define TSP_CUDA(call)                                                                              \
    do {                                                                                            \
        cudaError_t e__ = (call);                                                                   \
        if (e__ != cudaSuccess) {                                                                   \
            tsp_set_error("%s:%d %s -> %s", __FILE__, __LINE__, #call, cudaGetErrorString(e__));    \
            return e__ == cudaErrorMemoryAllocation ? TSP_ENOMEM : TSP_ECUDA;                       \
        }                                                                                           \
    } while (0)

#define TSP_TRY(call)                  \
    do {                               \
        int rc__ = (call);             \
        if (rc__ != TSP_OK) return rc__; \
    } while (0)

// ---------------------------------------------------------------- tile geometry and layouts

__host__ __device__ inline int tsp_bm(int cls) { return cls == 0 ? 64 : (cls == 1 ? 16 : 8); }
__host__ __device__ inline int tsp_bn(int precision, int cls)
{
    return precision == 0 ? (cls == 0 ? 32 : 16) : (cls == 0 ? 16 : 8);
}

// Position of element (r, c) of a 16 x KW block in mma.sync A-fragment order (KW = 16 FP16 / 8 TF32):
// lane l = (r%8)*4 + ..., each lane owns 8 halves / 4 floats.  This is the order upstream stores 16-row
// tiles in (src/csr2tile.h:289-307) and the order one 16-byte load per lane wants.
__host__ __device__ inline int tsp_frag16_index(int precision, int r, int c)
{
    if (precision == 0) return ((((r & 7) << 2) + ((c & 7) >> 1)) << 3) + ((c >> 3) << 2) + ((r >> 3) << 1) + (c & 1);
    return ((((r & 7) << 2) + (c & 3)) << 2) + ((c >> 2) << 1) + (r >> 3);
}

// Position of (r, c) inside one tile in the upstream layout (src/csr2tile.h:255-373).
__host__ __device__ inline int tsp_upstream_index(int precision, int cls, int r, int c)
{
    if (cls == 2)  // 8-row tile = the k x n8 operand of the MMA (src/csr2tile.h:262-271)
    {
        if (precision == 0) return (((r << 2) + ((c >> 1) & 3)) << 2) + ((c >> 3) << 1) + (c & 1);
        return (((r << 2) + (c & 3)) << 1) + (c >> 2);
    }
    if (cls == 1) return tsp_frag16_index(precision, r, c);
    const int KW = precision == 0 ? 16 : 8;  // 64-row: 4 x 2 sub-blocks, sub_m-major (src/csr2tile.h:319-372)
    return ((r >> 4) * 2 + c / KW) * 16 * KW + tsp_frag16_index(precision, r & 15, c % KW);
}

// Position (in elements) of (r, k) inside one 64-row tile as the DEVICE keeps it: the K-major, no-swizzle
// shared-memory operand layout of tcgen05.mma.  A core matrix is 8 rows x 16 bytes (T = 8 halves / 4 floats),
// stored as 128 contiguous bytes; core matrix (mi = r/8, ki = k/T) sits at byte (ki*8 + mi)*128, so that one
// K-slice of an MMA (two core-matrix columns, 2 KB) is contiguous and a whole tile is one 4 KB bulk copy.
__host__ __device__ inline int tsp_umma_index(int precision, int r, int k)
{
    const int T = precision == 0 ? 8 : 4;
    return ((k / T) * 8 + (r >> 3)) * 8 * T + (r & 7) * T + (k % T);
}

// Position of (r, c) in the layout the device stores for class cls.
__host__ __device__ inline int tsp_device_index(int precision, int cls, int r, int c)
{
    return cls == 0 ? tsp_umma_index(precision, r, c) : tsp_upstream_index(precision, cls, r, c);
}

// A 64-row tile with at most this many distinct entries is kept as a packed record (row masks + values), a fuller one
// as a dense 4 KB tile.
#define TSP_REC_MAX_VALS(PREC) ((PREC) == 0 ? 256 : 128)
__host__ __device__ inline int tsp_mask_bytes(int precision) { return precision == 0 ? 256 : 128; }
// A packed record holds n_pad = n rounded up to 8 entries: n_pad 16-bit positions (the element index of the value in
// the 4 KB operand tile, tsp_umma_index; 0xffff in the padding) followed by n_pad values.  Size in 16-byte units:
__host__ __device__ inline unsigned int tsp_packed_units(int precision, int n)
{
    return (unsigned int)(((n + 7) & ~7) * (2 + (precision ? 4 : 2))) / 16u;
}

// Width of the column stripe one task unit covers for (class, padded dense width): the 64-row kernel keeps up to
// 256 accumulator columns in tensor memory, the 16/8-row kernels up to 128 in registers.
__host__ __device__ inline int tsp_stripe_width(int cls, int colB)
{
    if (colB == 32) return 32;
    if (cls == 0) return colB % 256 == 0 ? 256 : (colB % 128 == 0 ? 128 : 64);
    return colB % 128 == 0 ? 128 : 64;
}

// ---------------------------------------------------------------- tracing and the checked build

// NVTX ranges (header-only; a no-op unless a profiler is attached) around conversion stages, scheduling and the class
// kernels, so that a timeline shows the same phases this library reports.
#include <nvtx3/nvToolsExt.h>
struct TspRange
{
    explicit TspRange(const char *name) { nvtxRangePushA(name); }
    ~TspRange() { nvtxRangePop(); }
};

// What a kernel needs to check its own indices in the checked build (-DTSP_DEBUG, libtilespmm_b200_debug.so): every
// gathered B row must lie inside B, every task inside the class's tiles, every written C row inside the caller's C.
// A violation is recorded in the handle's error flag (codes 0x20..0x22, reported as TSP_EINVAL by tsp_check_error) and
// the access is skipped or redirected to row 0 -- never performed.  The release build passes the struct and ignores it.
struct TspBounds
{
    int colA, tilenum, c_rows;
};
#ifdef TSP_DEBUG
#define TSP_CHECKED 1
#else
#define TSP_CHECKED 0
#endif

// ---------------------------------------------------------------- handle

struct TspKernelResources  // what the platform probe records per (class, width) kernel
{
    int threads, registers_per_thread, iteration_bytes, tasks_per_block;
    long long shared_bytes;
};

struct TspClass
{
    int BM = 0, BN = 0;
    int rows = 0;            // rows of the shard assigned to this class
    long long nnz = 0;
    int tilem = 0, tilenum = 0;
    int *d_tile_ptr = nullptr, *d_tile_nnz = nullptr, *d_tile_colidx = nullptr, *d_panel_row = nullptr;
    void *d_val = nullptr;          // dense tiles of the 16- and 8-row classes (upstream fragment order); unused for 64-row tiles
    // 64-row class only: packed tile records (see spmm64.cu).  d_bitmap[tile][row] = column mask of the row inside the
    // tile (uint16 for TF32 tiles of 16 columns, uint32 for FP16 tiles of 32 columns); d_rec[tile] = offset of the
    // tile's record in d_pack in 16-byte units, bit 31 set when the record is a dense 4 KB tile; d_rec[tilenum] = end.
    void *d_bitmap = nullptr;
    unsigned int *d_rec = nullptr;
    unsigned char *d_pack = nullptr;
    long long pack_bytes = 0;
    std::vector<int> h_tile_ptr, h_panel_row;
    // schedule for the current threshold
    int TH = 0, ntasks = 0, nsplit = 0;
    long long cap_tasks = 0, cap_panels = 0;   // capacities of the task arrays / the per-panel arrays (kept across conversions)
    unsigned int *d_task_row = nullptr;
    int *d_task_start = nullptr, *d_split_row = nullptr, *d_task_count = nullptr;
    // the same tasks as {row word, first tile, end tile, 0}, longest first (what the 16/8-row kernels walk)
    uint4 *d_task_pack = nullptr;
};

struct tsp_handle
{
    int device = 0, precision = 0;
    cudaDeviceProp prop;
    int rowA = 0, colA = 0;
    long long nnzA = 0;
    bool converted = false;
    int row_begin = 0, row_end = 0;   // C slab of this shard (original rows)
    TspClass cls[3];
    cudaStream_t side[2] = {nullptr, nullptr};
    cudaEvent_t fork = nullptr, join[2] = {nullptr, nullptr};
    cudaEvent_t t0 = nullptr, t1 = nullptr;
    long long launches = 0;
    int *d_error = nullptr;           // device-side error flag (bounded waits)
    // all tile arrays of the three classes live in two allocations (the second holds the packed 64-row records)
    void *tile_block = nullptr, *pack_block = nullptr;
    size_t tile_block_bytes = 0, pack_block_bytes = 0;   // capacities: a later conversion that fits reuses the allocation
    // conversion workspace: chunks of device memory reused by every conversion of this handle, and a small pinned
    // host buffer for the few scalars a conversion reads back
    std::vector<std::pair<void *, size_t>> ws_chunks;
    void *h_pin = nullptr;
    // device staging of the host-buffer entry points: two slots, so that the upload of one call overlaps the
    // download of the previous one (PCIe is full duplex); one stream per direction plus a compute stream
    void *stage_b[2] = {nullptr, nullptr};
    float *stage_c[2] = {nullptr, nullptr};
    size_t stage_b_bytes[2] = {0, 0}, stage_c_bytes[2] = {0, 0};
    cudaStream_t s_in = nullptr, s_cmp = nullptr, s_out = nullptr;
    cudaEvent_t ev_in[2] = {nullptr, nullptr}, ev_cmp[2] = {nullptr, nullptr}, ev_out[2] = {nullptr, nullptr};
    bool slot_busy[2] = {false, false};
    // tensor map over B for the gather4 loads of the 64-row kernel, rebuilt when B's address or width changes
    alignas(64) unsigned char bmap[128];
    const void *bmap_ptr = nullptr;
    int bmap_cols = 0, bmap_box = 0;
};

// ---------------------------------------------------------------- cross-TU entry points

// rowptr/colidx/val are device pointers, or host pointers when csr_on_host (uploaded into the conversion workspace)
int tsp_convert_impl(tsp_handle *h, int rowA, int colA, long long nnz, const int *rowptr, const int *colidx, const void *val,
                     bool csr_on_host, float gamma, float delta, int shard_index, int shard_count);
// forgets the converted matrix; release = false keeps the device allocations for the next conversion
void tsp_free_tiles(tsp_handle *h, bool release = false);
int tsp_export_values_upstream(const tsp_handle *h, int cls, void *h_dst);
// one allocation for the tile arrays of all classes (sizes from cls[k].tilem / tilenum), zero-filled where needed
int tsp_alloc_tile_arrays(tsp_handle *h);
int tsp_alloc_pack(tsp_handle *h, long long bytes);
void tsp_free_workspace(tsp_handle *h);

// class kernels; C is addressed relative to row_begin.  count_only != 0 skips the launch and only reports
// how many launches the call would make.
int tsp_launch_class64(tsp_handle *h, const void *d_b, float *d_c, int colB, cudaStream_t s);
int tsp_launch_class64_tma(tsp_handle *h, const void *d_b, float *d_c, int colB, cudaStream_t s);
int tsp_launch_small(tsp_handle *h, int cls, const void *d_b, float *d_c, int colB, cudaStream_t s);
int tsp_launch_small_t(tsp_handle *h, int cls, const void *d_b, float *d_c, int colB, cudaStream_t s);
bool tsp_small_t_supported(int colB);
int tsp_launch_clear(tsp_handle *h, float *d_c, int colB, cudaStream_t s);
int tsp_launch_selftest_wait(tsp_handle *h, unsigned polls, cudaStream_t s);
void tsp_kernel_resources(int precision, int cls, int colB, TspKernelResources *out);
inline TspBounds tsp_bounds(const tsp_handle *h, int cls)
{
    return TspBounds{h->colA, h->cls[cls].tilenum, (int)(((long long)(h->row_end - h->row_begin) + 64) / 64 * 64)};
}
