/*
 * tilespmm_b200 -- C ABI of the B200-native TileSpMM hot path (libtilespmm_b200.so).
 *
 * The upstream project (SuperScientificSoftwareLaboratory/TileSpMM) has no library API: its surface is two
 * executables plus header-level C++ functions compiled into them.  Each entry point below replaces one of
 * those functions; the comment above it names the upstream file:line it stands in for.  All functions
 * return 0 on success and a positive TSP_E* code otherwise (upstream prints and exits instead,
 * src/common.h:75-94); tsp_last_error() returns the message of the last failure on the calling thread.
 *
 * Conventions: precision 0 = FP16 values (IEEE binary16 bit patterns), precision 1 = TF32 (plain float,
 * the tensor core ignores the low 13 mantissa bits exactly as in upstream, src/tilespmm_cuda.h:1118-1124).
 * Tile classes: 0 = 64-row panels, 1 = 16-row panels, 2 = 8-row panels.  Tile widths (K extent) are
 * 32/16/16 for FP16 and 16/8/8 for TF32 (src/main.cu:267-275).  All index arrays are 32-bit like upstream
 * (src/common.h:34-36).  Pointers named h_* are host memory, d_* are device memory on the handle's device.
 */
#ifndef TILESPMM_B200_H
#define TILESPMM_B200_H

#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct tsp_handle tsp_handle;

enum
{
    TSP_OK = 0,
    TSP_EINVAL = 1,    /* bad argument */
    TSP_ECUDA = 2,     /* a CUDA call failed */
    TSP_ENOMEM = 3,    /* host or device allocation failed */
    TSP_ESTATE = 4,    /* call order violated (e.g. spmm before convert) */
    TSP_EDEVICE = 5,   /* the device is not an sm_100 part */
    TSP_ETIMEOUT = 6   /* a bounded device-side wait ran out; the kernel returned early */
};

const char *tsp_last_error(void);
int tsp_version(void);

/* ---- threshold model.  Same C ABI as upstream lib/model.so (src/ml_predict.h:8-15): 11 doubles in
 * {unused, unused, rows, cols, nnz, sparsity, avg_row_nnz, max_row_nnz, min_row_nnz, capability, colB},
 * (gamma, delta) out.  The decision table is re-derived for B200 and these kernels. */
void tilespmm_predict_fp16(const double *features, float *gamma, float *delta);
void tilespmm_predict_tf32(const double *features, float *gamma, float *delta);
/* The same walk (upstream tilespmm_policy_select, src/model.h:3463-3491) over a caller-supplied table of `nnodes` nodes
 * of 11 32-bit fields each, {feature, left_feature, right_feature, child0..3, missing_left_mask, cut, left_cut,
 * right_cut} (src/model.h:9-13), starting at `root`; a negative child -1-a is the leaf of candidate a.  For checking a
 * refitted table before it is compiled in.  TSP_EINVAL when the table is malformed. */
int tsp_policy_walk(const void *nodes, int nnodes, int root, const double *features11, float *gamma, float *delta);
/* upstream features_from_csr (src/model_features.h:31-57); returns 0 when the CSR is inconsistent. */
int tsp_features_from_csr(int rows, int cols, long long nnz, const int *h_rowptr, double capability, int colB,
                          double *features11);

/* ---- handle.  One handle owns one converted matrix on one device. */
int tsp_create(tsp_handle **out, int device, int precision);
int tsp_destroy(tsp_handle *h);

/* ---- partition + conversion on the GPU: upstream matrix_split (src/hetero_split.h:144-291) followed by the
 * three Tile_create calls (src/csr2tile.h:724-795, src/main.cu:266-275).  The CSR may be unsorted within
 * rows and may hold repeated (row, col) entries, which are summed in value type in CSR order.
 * shard_index/shard_count: only the panels of this shard (a contiguous range of the global panel sequence,
 * balanced by tile bytes) are converted -- 0/1 converts everything.  The partition itself is always global,
 * so shards of one matrix agree with the unsharded tiling. */
int tsp_convert_host(tsp_handle *h, int rowA, int colA, long long nnz, const int *h_rowptr, const int *h_colidx,
                     const void *h_val, float gamma, float delta, int shard_index, int shard_count);
int tsp_convert_device(tsp_handle *h, int rowA, int colA, long long nnz, const int *d_rowptr, const int *d_colidx,
                       const void *d_val, float gamma, float delta, int shard_index, int shard_count);

/* info12[c*4 + {0,1,2,3}] = rows, nnz, panels (tilem), tiles (tilenum) of class c -- the quantities upstream
 * prints into its CSV row (src/main.cu:306-307); all fit an int because the whole matrix is limited to 2^31-1 entries.  shard_rows[2] = first and one-past-last original row of
 * the C slab this handle writes. */
int tsp_info(const tsp_handle *h, int *info12, int *shard_rows2);

/* Copies one tiling array to host memory in UPSTREAM layout (src/format.h:4-21): which = 0 orig_row[rows],
 * 1 tile_ptr[tilem+1], 2 tile_nnz[tilenum+1], 3 tile_colidx[tilenum*BN], 4 Blockdense_Val[tilenum*BM*BN]
 * (the device keeps 64-row tiles as packed records; the export expands them to upstream's dense tiles),
 * 5 orig_tile_row_idx[tilem].  Arrays with no upstream counterpart, 64-row class only (cls 0): 6 the row masks,
 * [tilenum][64] words of 16 bits (TF32) or 32 bits (FP16), bit k of word r set when position (r, k) of the tile holds
 * a stored entry (an explicit zero counts); 7 rec[tilenum+1], offset of every tile's record in 16-byte units with bit
 * 31 set for a dense record; 8 the records: a packed record of a tile with n entries is n rounded up to 8 positions
 * of 16 bits (the entry's element index in the 4 KB tcgen05 operand tile, 0xffff in the padding) followed by as many
 * values, both in row-major order of the set mask bits; a dense record (more than 128 TF32 / 256 FP16 entries) is the
 * 4 KB tile in tcgen05 core-matrix order.  h_dst == NULL only queries the size.  *bytes receives the size. */
int tsp_export(const tsp_handle *h, int cls, int which, void *h_dst, long long *bytes);

/* ---- load balancing.  upstream get_optimal_prefetch_th (src/csr2tile.h:437-642) with the resource table of
 * THESE kernels (probed with cudaFuncGetAttributes at tsp_create, the role of upstream pre/prefetch_probe.cu). */
int tsp_top4(const tsp_handle *h, int cls, int colB_padded, int *top4);
/* The resource row of the kernel that serves (cls, colB_padded) on this device -- what upstream's platform probe
 * prints per kernel (pre/prefetch_probe.cu:12-28): out6 = {threads per block, registers per thread, shared bytes
 * per block, bytes fetched per pipeline step of a block, tasks per block, column stripes per task}. */
int tsp_kernel_info(const tsp_handle *h, int cls, int colB_padded, long long *out6);
/* The weight of one atomic slice that tsp_top4 uses for (precision, cls, colB_padded): the platform calibration that
 * upstream hard-codes as the lambda_atom table of get_optimal_prefetch_th (src/csr2tile.h:483-495), here fitted to
 * these kernels on B200 (tilespmm_b200/calibrate_atom.py writes csrc/atom_table.inc). */
float tsp_atom_weight(int precision, int cls, int colB_padded);
/* upstream tile_pretreatment + update_metadata (src/csr2tile.h:383-434, 644-711): builds the task arrays of
 * class cls for threshold TH on the device. */
int tsp_schedule(tsp_handle *h, int cls, int TH);
/* No counterpart in upstream.  The same task arrays as tsp_schedule(), built without cudaMalloc/cudaFree or
 * any allocating library call, for hosts that own all device memory themselves (a pre-carved arena) or may
 * not enter the allocator on their hot path.  The per-panel counters live in a fixed device array inside
 * the library (4 MB + 260 bytes per GPU, held until the process exits), so tilem is limited to 1,048,576 panels
 * (TSP_EINVAL beyond that).  Inputs d_tile_ptr[tilem+1], d_panel_row[tilem]; outputs d_task_row[capacity],
 * d_task_start[capacity+1], d_split_row[tilem] (may be NULL) are caller-owned device arrays; *ntasks and
 * *nsplit are host outputs.  TSP_ENOMEM (with *ntasks = tasks needed, nothing written) when capacity is too
 * small.  The first call on a device resolves the array's device address and loads the kernels (both may allocate
 * inside the CUDA runtime): make it at start-up, before any stream capture and before the arena is carved.  The
 * caller's current device is restored on return.
 * Calls share the array: back-to-back calls are fine, calls that can overlap on one GPU race.  Waits for
 * `stream` before returning. */
int tsp_schedule_noalloc(int device, int tilem, int TH, const int *d_tile_ptr, const int *d_panel_row,
                         unsigned int *d_task_row, int *d_task_start, long long capacity, int *d_split_row,
                         int *ntasks, int *nsplit, void *stream);
/* Current task arrays: rows[ntasks] (bit 31 = slice of a split panel), colstart[ntasks+1]; NULL = count only. */
int tsp_export_schedule(const tsp_handle *h, int cls, int *ntasks, unsigned int *h_rows, int *h_colstart);
/* On-GPU threshold tuning, upstream src/csr2tile.h:964-1019: every combination of the candidate thresholds,
 * 5 warm-up + 10 timed passes each; leaves the best schedules installed.  best3 = {th64, th16, th8}. */
int tsp_tune(tsp_handle *h, const void *d_b, float *d_c, int colB_padded, int *best3, float *tune_ms);

/* ---- SpMM.  C[rows of this shard, 0..colB_padded) = A * B with FP32 accumulation.  d_b is colA x colB_padded
 * row-major (value type), d_c is row-major float with row stride colB_padded and at least
 * tsp_c_rows() rows (upstream pads C to (rowA+64)/64*64 rows, src/csr2tile.h:835-842).  Unlike upstream
 * (src/csr2tile.h:1024) the caller does not have to clear C: panels without tiles are written as zeros and
 * the rows of split panels are cleared by a kernel of this call.  stream is a cudaStream_t (NULL = legacy). */
int tsp_spmm(tsp_handle *h, const void *d_b, float *d_c, int colB_padded, void *stream);
/* tsp_spmm only enqueues.  The tcgen05 kernels bound every device-side wait (upstream's kernels have none); when one
 * runs out the kernel records it, frees its tensor memory and returns early, leaving its part of C incomplete.
 * tsp_check_error waits for `stream` (NULL: the whole device) and returns TSP_ETIMEOUT if that happened in any launch
 * of this handle since the last check, TSP_OK otherwise; it clears the record.  The host-buffer entry points below,
 * tsp_time, tsp_tune and tsp_run check by themselves. */
int tsp_check_error(tsp_handle *h, void *stream);
/* Failure-path self test (no upstream counterpart): runs a one-block kernel that allocates tensor memory and waits
 * `polls` (1..2^22) polls on an mbarrier nobody arrives on, gives up, frees the tensor memory and returns.  The call
 * must return TSP_ETIMEOUT and leave the handle fully usable; nothing hangs, traps or faults. */
int tsp_selftest_wait_timeout(tsp_handle *h, int polls);
long long tsp_c_rows(const tsp_handle *h);
/* Same, with host buffers: copies B to the device, runs, copies the first rowA rows of C back
 * (upstream src/csr2tile.h:839-842, 1020-1032). */
int tsp_spmm_host(tsp_handle *h, const void *h_b, float *h_c, int colB_padded);
/* The same in two steps, for callers that stream many right-hand sides: _async starts upload, kernels and download in
 * staging slot 0 or 1 and returns; _wait blocks until C of that slot is in h_c.  Alternating the slots overlaps the
 * upload of one call with the download of the previous one.  Buffers must stay valid (ideally pinned) until _wait. */
int tsp_spmm_host_async(tsp_handle *h, const void *h_b, float *h_c, int colB_padded, int slot);
int tsp_spmm_host_wait(tsp_handle *h, int slot);

/* Kernel launches issued by tsp_spmm so far (all classes, including the clearing kernel). */
long long tsp_launch_count(const tsp_handle *h);
/* Algorithmic bytes of one SpMM in the upstream tile format: bytes3 = {A tiles + column indices, gathered B
 * rows, C}; per class when cls >= 0, all classes when cls < 0. */
int tsp_algorithmic_bytes(const tsp_handle *h, int cls, int colB_padded, double *bytes3);
/* Bytes of the tile data as THIS library keeps it in device memory (what its kernels read per column stripe): dense
 * tiles of the 16/8-row classes, packed records of the 64-row class, column indices. */
int tsp_tile_bytes(const tsp_handle *h, int cls, double *bytes);
/* Times `iters` passes of one class kernel alone (cls 0..2) or of the whole SpMM (cls < 0) with CUDA events
 * on the launching stream; ms = mean per pass. */
int tsp_time(tsp_handle *h, int cls, const void *d_b, float *d_c, int colB_padded, int iters, float *ms);

/* ---- the upstream runtime driver call_tilespmm_cuda (src/csr2tile.h:826-1093): upload, threshold candidates,
 * warm-up, tuning, checked run (h_c receives rowA x colB_padded floats, may be NULL), timed loop of `repeat`
 * passes.  out6 = {best_th64, best_th16, best_th8, pre_time_ms (cpu_pre_time_ms + candidate + tuning time),
 * time_ms, tflops = 2*nnz*colB_logical/time}. */
int tsp_run(tsp_handle *h, const void *h_b, float *h_c, int colB_padded, int colB_logical, double cpu_pre_time_ms,
            int repeat, double *out6);

/* ---- several GPUs of one box inside one process (no upstream counterpart: upstream runs on the one GPU `-d` names,
 * src/main.cu:138-142, 210).  The panel sequence of the matrix is cut into contiguous ranges balanced by tile bytes, one
 * per device; every device converts and multiplies its range and owns the matching row slab of C.  B is uploaded in N
 * row blocks, one per device, and all-gathered over NCCL (loaded at run time; not needed for one device) into every
 * device's own memory; C is row-partitioned, no reduction.  The calls mirror the single-GPU ones above. */
typedef struct tsp_multi tsp_multi;
int tsp_multi_create(tsp_multi **out, int ndev, const int *devices, int precision);
int tsp_multi_destroy(tsp_multi *m);
int tsp_multi_device_count(const tsp_multi *m);
/* one host thread per device converts that device's shard (tsp_convert_host with shard i of ndev) */
int tsp_multi_convert_host(tsp_multi *m, int rowA, int colA, long long nnz, const int *h_rowptr, const int *h_colidx,
                           const void *h_val, float gamma, float delta);
/* info12 as tsp_info, summed over the devices; slabs2n[2i], slabs2n[2i+1] = rows of device i's slab of C (may be NULL) */
int tsp_multi_info(const tsp_multi *m, int *info12, int *slabs2n);
/* h_b: colA x colB_padded values; h_c: rowA x colB_padded floats */
int tsp_multi_spmm_host(tsp_multi *m, const void *h_b, float *h_c, int colB_padded);
/* tsp_run over the devices: per-device tuning, checked product (h_c may be NULL), `repeat` timed passes on all devices
 * together; out6 as tsp_run with the thresholds of device 0 and the slowest device's mean time */
int tsp_multi_run(tsp_multi *m, const void *h_b, float *h_c, int colB_padded, int colB_logical, double cpu_pre_time_ms,
                  int repeat, double *out6);

/* ---- the cuSPARSE baseline upstream runs next to its own kernels, cusparse_spmm_all (src/main.cu:16-134):
 * CSR, CUSPARSE_SPMM_ALG_DEFAULT, FP32 compute; FP16 inputs for precision 0 and true FP32 inputs for
 * precision 1.  h_c is m x n floats (may be NULL).  out3 = {pre_time_ms, time_ms, tflops}. */
int tsp_cusparse_baseline(int device, int precision, int m, int k, long long nnz, const int *h_rowptr,
                          const int *h_colidx, const void *h_val, int n, int ldb, const void *h_b, float *h_c,
                          int warmup, int repeat, double *out3);

/* The same measurement with another cuSPARSE algorithm: alg 0 = ALG_DEFAULT (what upstream runs), 1..3 =
 * CUSPARSE_SPMM_CSR_ALG1..3, with cusparseSpMM_preprocess counted in pre_time_ms.  A stronger baseline, reported
 * beside upstream's number, never instead of it. */
int tsp_cusparse_baseline_alg(int device, int precision, int m, int k, long long nnz, const int *h_rowptr,
                              const int *h_colidx, const void *h_val, int n, int ldb, const void *h_b, float *h_c,
                              int warmup, int repeat, int alg, double *out3);

/* ---- tile cache on disk (no upstream counterpart: upstream converts on every run).  tsp_save writes the converted
 * matrix of the handle (all classes, shard limits included) to one binary file; tsp_load restores it into a handle of
 * the same precision, replacing whatever it held, without touching the CSR again. */
int tsp_save(const tsp_handle *h, const char *path);
int tsp_load(tsp_handle *h, const char *path);

/* ---- Matrix Market loader with the semantics of upstream mmio_allinone (src/mmio_highlevel.h:307-480): file order
 * inside rows, repeated entries kept, symmetric/hermitian files expanded, pattern = 1.0.  The three arrays are
 * malloc'ed by the callee; release each with tsp_free_host. */
int tsp_read_mtx(const char *path, int *m, int *n, long long *nnz, int *is_symmetric, int **h_rowptr, int **h_colidx,
                 float **h_val);
void tsp_free_host(void *p);

#ifdef __cplusplus
}
#endif
#endif
