// C ABI of libtilespmm_b200.so: handle life cycle, conversion entry points, export, SpMM, timing, the
// runtime driver that mirrors upstream call_tilespmm_cuda (src/csr2tile.h:826-1093) and the cuSPARSE
// baseline that mirrors upstream cusparse_spmm_all (src/main.cu:16-134).
#include <cusparse.h>
#include <dlfcn.h>
#include <math.h>
#include <stdarg.h>
#include <stdlib.h>
#include <string.h>
#include <sys/time.h>

#include "tsp_internal.cuh"

static thread_local char g_error[512] = "";

void tsp_set_error(const char *fmt, ...)
{
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_error, sizeof(g_error), fmt, ap);
    va_end(ap);
}

extern "C" const char *tsp_last_error(void) { return g_error; }
extern "C" int tsp_version(void) { return 100; }

extern "C" int tsp_features_from_csr(int rows, int cols, long long nnz, const int *rp, double capability, int colB, double *f)
{
    // upstream features_from_csr / features_from_stats (src/model_features.h:8-57)
    if (!rp || !f || rows <= 0 || cols <= 0 || nnz < 0 || rp[0] != 0 || (long long)rp[rows] != nnz) return 0;
    if (!(capability > 0.0) || capability != capability || capability > 1e300 || colB <= 0) return 0;
    int mn = 0x7fffffff, mx = 0;
    for (int r = 0; r < rows; r++)
    {
        const long long cnt = (long long)rp[r + 1] - rp[r];
        if (cnt < 0) return 0;
        if (cnt < mn) mn = (int)cnt;
        if (cnt > mx) mx = (int)cnt;
    }
    f[0] = 0.0; f[1] = 0.0;
    f[2] = rows; f[3] = cols; f[4] = (double)nnz;
    f[5] = 1.0 - (double)nnz / ((double)rows * (double)cols);
    f[6] = (double)nnz / (double)rows;
    f[7] = mx; f[8] = mn; f[9] = capability; f[10] = colB;
    return 1;
}

static int create_resources(tsp_handle *h);

extern "C" int tsp_create(tsp_handle **out, int device, int precision)
{
    if (!out || (precision != 0 && precision != 1)) { tsp_set_error("create: bad argument"); return TSP_EINVAL; }
    *out = nullptr;
    int ndev = 0;
    cudaError_t e = cudaGetDeviceCount(&ndev);
    if (e != cudaSuccess || device < 0 || device >= ndev)
    {
        tsp_set_error("create: no CUDA device %d (%s)", device, e == cudaSuccess ? "out of range" : cudaGetErrorString(e));
        return TSP_ECUDA;
    }
    tsp_handle *h = new tsp_handle();
    h->device = device; h->precision = precision;
    const int rc = create_resources(h);
    if (rc != TSP_OK) { tsp_destroy(h); return rc; }
    *out = h;
    return TSP_OK;
}

static int create_resources(tsp_handle *h)
{
    const int device = h->device, precision = h->precision;
    TSP_CUDA(cudaSetDevice(device));
    TSP_CUDA(cudaGetDeviceProperties(&h->prop, device));
    if (h->prop.major != 10)
    {
        tsp_set_error("create: device %d is sm_%d%d; this library is built for sm_100a only", device, h->prop.major, h->prop.minor);
        return TSP_EDEVICE;
    }
    for (int k = 0; k < 3; k++) { h->cls[k].BM = tsp_bm(k); h->cls[k].BN = tsp_bn(precision, k); }
    for (int i = 0; i < 2; i++)
    {
        TSP_CUDA(cudaStreamCreateWithFlags(&h->side[i], cudaStreamNonBlocking));
        TSP_CUDA(cudaEventCreateWithFlags(&h->join[i], cudaEventDisableTiming));
    }
    TSP_CUDA(cudaEventCreateWithFlags(&h->fork, cudaEventDisableTiming));
    TSP_CUDA(cudaEventCreate(&h->t0));
    TSP_CUDA(cudaEventCreate(&h->t1));
    TSP_CUDA(cudaMalloc((void **)&h->d_error, 4));
    TSP_CUDA(cudaMemset(h->d_error, 0, 4));
    return TSP_OK;
}

extern "C" int tsp_destroy(tsp_handle *h)
{
    if (!h) return TSP_OK;
    cudaSetDevice(h->device);
    cudaDeviceSynchronize();
    tsp_free_tiles(h, true);
    tsp_free_workspace(h);
    if (h->h_pin) cudaFreeHost(h->h_pin);
    for (int i = 0; i < 2; i++) { if (h->side[i]) cudaStreamDestroy(h->side[i]); if (h->join[i]) cudaEventDestroy(h->join[i]); }
    if (h->fork) cudaEventDestroy(h->fork);
    if (h->t0) cudaEventDestroy(h->t0);
    if (h->t1) cudaEventDestroy(h->t1);
    cudaFree(h->d_error);
    for (int i = 0; i < 2; i++)
    {
        cudaFree(h->stage_b[i]); cudaFree(h->stage_c[i]);
        if (h->ev_in[i]) cudaEventDestroy(h->ev_in[i]);
        if (h->ev_cmp[i]) cudaEventDestroy(h->ev_cmp[i]);
        if (h->ev_out[i]) cudaEventDestroy(h->ev_out[i]);
    }
    if (h->s_in) { cudaStreamDestroy(h->s_in); cudaStreamDestroy(h->s_cmp); cudaStreamDestroy(h->s_out); }
    delete h;
    return TSP_OK;
}

extern "C" int tsp_convert_device(tsp_handle *h, int rowA, int colA, long long nnz, const int *d_rowptr, const int *d_colidx,
                                  const void *d_val, float gamma, float delta, int shard_index, int shard_count)
{
    if (!h || !d_rowptr || (nnz > 0 && (!d_colidx || !d_val))) { tsp_set_error("convert: null argument"); return TSP_EINVAL; }
    return tsp_convert_impl(h, rowA, colA, nnz, d_rowptr, d_colidx, d_val, false, gamma, delta, shard_index, shard_count);
}

extern "C" int tsp_convert_host(tsp_handle *h, int rowA, int colA, long long nnz, const int *rp, const int *ci, const void *val,
                                float gamma, float delta, int shard_index, int shard_count)
{
    if (!h || !rp || rowA <= 0 || nnz < 0 || (nnz > 0 && (!ci || !val))) { tsp_set_error("convert: bad argument"); return TSP_EINVAL; }
    return tsp_convert_impl(h, rowA, colA, nnz, rp, ci, val, true, gamma, delta, shard_index, shard_count);
}

extern "C" int tsp_info(const tsp_handle *h, int *info12, int *shard_rows2)
{
    if (!h || !info12) { tsp_set_error("info: null argument"); return TSP_EINVAL; }
    for (int k = 0; k < 3; k++)
    {
        info12[k * 4 + 0] = h->cls[k].rows;
        info12[k * 4 + 1] = (int)h->cls[k].nnz;
        info12[k * 4 + 2] = h->cls[k].tilem;
        info12[k * 4 + 3] = h->cls[k].tilenum;
    }
    if (shard_rows2) { shard_rows2[0] = h->row_begin; shard_rows2[1] = h->row_end; }
    return TSP_OK;
}

extern "C" int tsp_export(const tsp_handle *h, int cls, int which, void *dst, long long *bytes)
{
    if (!h || cls < 0 || cls > 2 || !bytes) { tsp_set_error("export: bad argument"); return TSP_EINVAL; }
    if (!h->converted) { tsp_set_error("export: convert first"); return TSP_ESTATE; }
    TSP_CUDA(cudaSetDevice(h->device));
    const TspClass &c = h->cls[cls];
    const size_t vsz = h->precision ? 4 : 2;
    *bytes = 0;
    if (c.rows == 0 && which != 7) return TSP_OK;
    switch (which)
    {
    case 0:  // orig_row: the rows of every panel, in panel order (src/hetero_split.h:86-141)
        *bytes = (long long)c.rows * 4;
        if (dst)
        {
            int *o = (int *)dst, n = 0;
            for (int p = 0; p < c.tilem; p++)
                for (int r = c.h_panel_row[p]; r < c.h_panel_row[p] + c.BM && r < h->rowA; r++) o[n++] = r;
        }
        return TSP_OK;
    case 1:
        *bytes = ((long long)c.tilem + 1) * 4;
        if (dst) memcpy(dst, c.h_tile_ptr.data(), (size_t)*bytes);
        return TSP_OK;
    case 2:
        *bytes = ((long long)c.tilenum + 1) * 4;
        if (dst) TSP_CUDA(cudaMemcpy(dst, c.d_tile_nnz, (size_t)*bytes, cudaMemcpyDeviceToHost));
        return TSP_OK;
    case 3:
        *bytes = (long long)c.tilenum * c.BN * 4;
        if (dst && *bytes) TSP_CUDA(cudaMemcpy(dst, c.d_tile_colidx, (size_t)*bytes, cudaMemcpyDeviceToHost));
        return TSP_OK;
    case 4:
        *bytes = (long long)c.tilenum * c.BM * c.BN * (long long)vsz;
        if (dst && *bytes) return tsp_export_values_upstream(h, cls, dst);
        return TSP_OK;
    case 5:
        *bytes = (long long)c.tilem * 4;
        if (dst) memcpy(dst, c.h_panel_row.data(), (size_t)*bytes);
        return TSP_OK;
    case 6:  // 64-row class: row masks of every tile
        if (cls != 0) return TSP_OK;
        *bytes = (long long)c.tilenum * tsp_mask_bytes(h->precision);
        if (dst && *bytes) TSP_CUDA(cudaMemcpy(dst, c.d_bitmap, (size_t)*bytes, cudaMemcpyDeviceToHost));
        return TSP_OK;
    case 7:  // 64-row class: record offsets
        if (cls != 0) return TSP_OK;
        *bytes = ((long long)c.tilenum + 1) * 4;
        if (dst && c.tilenum) TSP_CUDA(cudaMemcpy(dst, c.d_rec, (size_t)*bytes, cudaMemcpyDeviceToHost));
        else if (dst) memset(dst, 0, (size_t)*bytes);
        return TSP_OK;
    case 8:  // 64-row class: the records
        if (cls != 0) return TSP_OK;
        *bytes = c.pack_bytes;
        if (dst && *bytes) TSP_CUDA(cudaMemcpy(dst, c.d_pack, (size_t)*bytes, cudaMemcpyDeviceToHost));
        return TSP_OK;
    default:
        tsp_set_error("export: unknown array %d", which);
        return TSP_EINVAL;
    }
}

extern "C" int tsp_kernel_info(const tsp_handle *h, int cls, int colB, long long *out6)
{
    if (!h || cls < 0 || cls > 2 || !out6 || colB <= 0) { tsp_set_error("kernel_info: bad argument"); return TSP_EINVAL; }
    TSP_CUDA(cudaSetDevice(h->device));
    TspKernelResources R;
    tsp_kernel_resources(h->precision, cls, colB, &R);
    const int stripe = tsp_stripe_width(cls, colB);
    out6[0] = R.threads; out6[1] = R.registers_per_thread; out6[2] = R.shared_bytes; out6[3] = R.iteration_bytes;
    out6[4] = R.tasks_per_block; out6[5] = colB / stripe;
    return TSP_OK;
}

extern "C" long long tsp_c_rows(const tsp_handle *h)
{
    if (!h) return 0;
    return ((long long)(h->row_end - h->row_begin) + 64) / 64 * 64;  // src/csr2tile.h:835
}

extern "C" long long tsp_launch_count(const tsp_handle *h) { return h ? h->launches : 0; }

static int check_width(int colB)
{
    if (colB == 32 || (colB > 0 && colB % 64 == 0)) return TSP_OK;  // src/main.cu:173
    tsp_set_error("the padded dense width must be 32 or a multiple of 64 (got %d)", colB);
    return TSP_EINVAL;
}

static int ensure_schedules(tsp_handle *h, int colB)
{
    for (int k = 0; k < 3; k++)
    {
        TspClass &c = h->cls[k];
        if (c.tilem > 0 && c.TH == 0)
        {
            int top4[4];
            TSP_TRY(tsp_top4(h, k, colB, top4));
            TSP_TRY(tsp_schedule(h, k, top4[0]));
        }
    }
    return TSP_OK;
}

static int launch_class(tsp_handle *h, int k, const void *d_b, float *d_c, int colB, cudaStream_t s)
{
    if (k != 0)
    {
        static int small_t = -1;   // TSP_SMALL=t selects the transposed tcgen05 kernel for the 16/8-row classes
        if (small_t < 0) { const char *e = getenv("TSP_SMALL"); small_t = (e && strcmp(e, "t") == 0) ? 1 : 0; }
        if (small_t && tsp_small_t_supported(colB)) return tsp_launch_small_t(h, k, d_b, d_c, colB, s);
        return tsp_launch_small(h, k, d_b, d_c, colB, s);
    }
    static int use_tma = -1;   // TSP_SPMM64=tma selects the TMA gather4 producer instead of the (faster) cp.async producers
    if (use_tma < 0) { const char *e = getenv("TSP_SPMM64"); use_tma = (e && strcmp(e, "tma") == 0) ? 1 : 0; }
    return use_tma ? tsp_launch_class64_tma(h, d_b, d_c, colB, s) : tsp_launch_class64(h, d_b, d_c, colB, s);
}

static int spmm_on(tsp_handle *h, const void *d_b, float *d_c, int colB, cudaStream_t s)
{
    TSP_TRY(tsp_launch_clear(h, d_c, colB, s));
    int active[3], na = 0;
    for (int k = 0; k < 3; k++) if (h->cls[k].ntasks > 0) active[na++] = k;
    if (na == 0) return TSP_OK;
    if (na > 1)
    {
        TSP_CUDA(cudaEventRecord(h->fork, s));
        for (int i = 1; i < na; i++) TSP_CUDA(cudaStreamWaitEvent(h->side[i - 1], h->fork, 0));
    }
    for (int i = 0; i < na; i++) TSP_TRY(launch_class(h, active[i], d_b, d_c, colB, i == 0 ? s : h->side[i - 1]));
    for (int i = 1; i < na; i++)
    {
        TSP_CUDA(cudaEventRecord(h->join[i - 1], h->side[i - 1]));
        TSP_CUDA(cudaStreamWaitEvent(s, h->join[i - 1], 0));
    }
    return TSP_OK;
}

static int check_device_error(tsp_handle *h)
{
    int flag = 0;
    TSP_CUDA(cudaMemcpy(&flag, h->d_error, 4, cudaMemcpyDeviceToHost));
    if (flag)
    {
        cudaMemset(h->d_error, 0, 4);
        if (flag >= 0x20 && flag <= 0x22)   // only the checked build (-DTSP_DEBUG) produces these
        {
            tsp_set_error("checked build: %s (code 0x%x); the access was skipped and the result of that launch is incomplete",
                          flag == 0x20 ? "a tile names a column outside B" : (flag == 0x21 ? "a task lies outside the class's tiles" : "a task writes rows outside C"), flag);
            return TSP_EINVAL;
        }
        if (flag == 4)
        {
            tsp_set_error("the shared memory of an SpMM kernel did not start on the boundary its operand layout needs; nothing was computed");
            return TSP_ECUDA;
        }
        tsp_set_error("a bounded wait inside an SpMM kernel ran out (code 0x%x); the result of that launch is incomplete", flag);
        return TSP_ETIMEOUT;
    }
    return TSP_OK;
}

// Waits for `stream` (NULL: the whole device) and reports a bounded wait that ran out in any kernel launched through
// this handle since the last check.  The flag is cleared, so the next call starts clean.
extern "C" int tsp_check_error(tsp_handle *h, void *stream)
{
    if (!h) { tsp_set_error("check_error: null handle"); return TSP_EINVAL; }
    TSP_CUDA(cudaSetDevice(h->device));
    if (stream) TSP_CUDA(cudaStreamSynchronize((cudaStream_t)stream));
    else TSP_CUDA(cudaDeviceSynchronize());
    return check_device_error(h);
}

#ifdef TSP_DEBUG
// Checked build only (libtilespmm_b200_debug.so): overwrites one index on the device so that the kernels' own checks can
// be exercised -- what 0: tile_colidx[index] of class cls, 1: the end tile of task `index` of class cls.  The release
// library does not have this entry point; its kernels never see a damaged index from this library's own conversion.
extern "C" int tsp_debug_poke(tsp_handle *h, int cls, int what, long long index, int value)
{
    if (!h || cls < 0 || cls > 2 || !h->converted || index < 0) { tsp_set_error("debug_poke: bad argument"); return TSP_EINVAL; }
    TSP_CUDA(cudaSetDevice(h->device));
    TspClass &c = h->cls[cls];
    if (what == 0)
    {
        if (index >= (long long)c.tilenum * c.BN) { tsp_set_error("debug_poke: index outside tile_colidx"); return TSP_EINVAL; }
        TSP_CUDA(cudaMemcpy(c.d_tile_colidx + index, &value, 4, cudaMemcpyHostToDevice));
    }
    else
    {
        if (index >= c.ntasks) { tsp_set_error("debug_poke: index outside the task list (schedule first)"); return TSP_EINVAL; }
        if (cls == 0) TSP_CUDA(cudaMemcpy(c.d_task_start + index + 1, &value, 4, cudaMemcpyHostToDevice));
        else TSP_CUDA(cudaMemcpy(&c.d_task_pack[index].z, &value, 4, cudaMemcpyHostToDevice));
    }
    return TSP_OK;
}
#endif

extern "C" int tsp_selftest_wait_timeout(tsp_handle *h, int polls)
{
    if (!h || polls <= 0 || polls > (1 << 22)) { tsp_set_error("selftest_wait_timeout: polls must be in 1..2^22"); return TSP_EINVAL; }
    TSP_CUDA(cudaSetDevice(h->device));
    TSP_TRY(tsp_launch_selftest_wait(h, (unsigned)polls, 0));
    return tsp_check_error(h, nullptr);
}

extern "C" int tsp_spmm(tsp_handle *h, const void *d_b, float *d_c, int colB, void *stream)
{
    if (!h || !d_b || !d_c) { tsp_set_error("spmm: null argument"); return TSP_EINVAL; }
    if (!h->converted) { tsp_set_error("spmm: convert first"); return TSP_ESTATE; }
    TSP_TRY(check_width(colB));
    TSP_CUDA(cudaSetDevice(h->device));
    TSP_TRY(ensure_schedules(h, colB));
    return spmm_on(h, d_b, d_c, colB, (cudaStream_t)stream);
}

// device staging buffers of the host-buffer entry points; they grow on demand and live as long as the handle
static int ensure_staging(tsp_handle *h, int slot, size_t b_bytes, size_t c_bytes)
{
    if (!h->s_in)
    {
        TSP_CUDA(cudaStreamCreateWithFlags(&h->s_in, cudaStreamNonBlocking));
        TSP_CUDA(cudaStreamCreateWithFlags(&h->s_cmp, cudaStreamNonBlocking));
        TSP_CUDA(cudaStreamCreateWithFlags(&h->s_out, cudaStreamNonBlocking));
        for (int i = 0; i < 2; i++)
        {
            TSP_CUDA(cudaEventCreateWithFlags(&h->ev_in[i], cudaEventDisableTiming));
            TSP_CUDA(cudaEventCreateWithFlags(&h->ev_cmp[i], cudaEventDisableTiming));
            TSP_CUDA(cudaEventCreateWithFlags(&h->ev_out[i], cudaEventDisableTiming));
        }
    }
    if (b_bytes > h->stage_b_bytes[slot])
    {
        cudaFree(h->stage_b[slot]); h->stage_b[slot] = nullptr; h->stage_b_bytes[slot] = 0;
        TSP_CUDA(cudaMalloc(&h->stage_b[slot], b_bytes));
        h->stage_b_bytes[slot] = b_bytes;
    }
    if (c_bytes > h->stage_c_bytes[slot])
    {
        cudaFree(h->stage_c[slot]); h->stage_c[slot] = nullptr; h->stage_c_bytes[slot] = 0;
        TSP_CUDA(cudaMalloc((void **)&h->stage_c[slot], c_bytes));
        h->stage_c_bytes[slot] = c_bytes;
    }
    return TSP_OK;
}

// Starts one SpMM with host buffers in staging slot 0 or 1 and returns without waiting: upload of B on the upload
// stream, kernels on the compute stream, download of C on the download stream, chained by events.  A caller that
// alternates the slots overlaps the upload of call i+1 with the download of call i.  h_b and h_c must stay valid
// (and should be pinned) until tsp_spmm_host_wait(h, slot) has returned.
extern "C" int tsp_spmm_host_async(tsp_handle *h, const void *h_b, float *h_c, int colB, int slot)
{
    if (!h || !h_b || !h_c || slot < 0 || slot > 1) { tsp_set_error("spmm_host_async: bad argument"); return TSP_EINVAL; }
    if (!h->converted) { tsp_set_error("spmm_host_async: convert first"); return TSP_ESTATE; }
    if (h->slot_busy[slot]) { tsp_set_error("spmm_host_async: slot %d is still in flight; call tsp_spmm_host_wait first", slot); return TSP_ESTATE; }
    TSP_TRY(check_width(colB));
    TSP_CUDA(cudaSetDevice(h->device));
    const size_t vsz = h->precision ? 4 : 2;
    const size_t b_bytes = (size_t)h->colA * colB * vsz, c_bytes = (size_t)tsp_c_rows(h) * colB * 4;
    TSP_TRY(ensure_staging(h, slot, b_bytes, c_bytes));
    TSP_TRY(ensure_schedules(h, colB));
    TSP_CUDA(cudaMemcpyAsync(h->stage_b[slot], h_b, b_bytes, cudaMemcpyHostToDevice, h->s_in));
    TSP_CUDA(cudaEventRecord(h->ev_in[slot], h->s_in));
    TSP_CUDA(cudaStreamWaitEvent(h->s_cmp, h->ev_in[slot], 0));
    TSP_TRY(spmm_on(h, h->stage_b[slot], h->stage_c[slot], colB, h->s_cmp));
    TSP_CUDA(cudaEventRecord(h->ev_cmp[slot], h->s_cmp));
    TSP_CUDA(cudaStreamWaitEvent(h->s_out, h->ev_cmp[slot], 0));
    TSP_CUDA(cudaMemcpyAsync(h_c, h->stage_c[slot], (size_t)(h->row_end - h->row_begin) * colB * 4, cudaMemcpyDeviceToHost, h->s_out));
    TSP_CUDA(cudaEventRecord(h->ev_out[slot], h->s_out));
    h->slot_busy[slot] = true;
    return TSP_OK;
}

extern "C" int tsp_spmm_host_wait(tsp_handle *h, int slot)
{
    if (!h || slot < 0 || slot > 1) { tsp_set_error("spmm_host_wait: bad argument"); return TSP_EINVAL; }
    if (!h->slot_busy[slot]) return TSP_OK;
    TSP_CUDA(cudaSetDevice(h->device));
    TSP_CUDA(cudaEventSynchronize(h->ev_out[slot]));
    h->slot_busy[slot] = false;
    return check_device_error(h);
}

extern "C" int tsp_spmm_host(tsp_handle *h, const void *h_b, float *h_c, int colB)
{
    TSP_TRY(tsp_spmm_host_async(h, h_b, h_c, colB, 0));
    return tsp_spmm_host_wait(h, 0);
}

extern "C" int tsp_algorithmic_bytes(const tsp_handle *h, int cls, int colB, double *b3)
{
    if (!h || !b3 || cls > 2) { tsp_set_error("algorithmic_bytes: bad argument"); return TSP_EINVAL; }
    const double vsz = h->precision ? 4 : 2;
    b3[0] = b3[1] = b3[2] = 0.0;
    for (int k = 0; k < 3; k++)
    {
        if (cls >= 0 && cls != k) continue;
        const TspClass &c = h->cls[k];
        b3[0] += (double)c.tilenum * (c.BM * c.BN * vsz + c.BN * 4.0);
        b3[1] += (double)c.tilenum * c.BN * colB * vsz;
        b3[2] += (double)c.rows * colB * 4.0;
    }
    return TSP_OK;
}

// Bytes of the tile data as this library stores it and as its kernels read it once per column stripe: values or
// records plus column indices; per class when cls >= 0, all classes when cls < 0.
extern "C" int tsp_tile_bytes(const tsp_handle *h, int cls, double *bytes)
{
    if (!h || !bytes || cls > 2) { tsp_set_error("tile_bytes: bad argument"); return TSP_EINVAL; }
    const double vsz = h->precision ? 4 : 2;
    *bytes = 0.0;
    for (int k = 0; k < 3; k++)
    {
        if (cls >= 0 && cls != k) continue;
        const TspClass &c = h->cls[k];
        *bytes += (double)c.tilenum * c.BN * 4.0 + (k == 0 ? (double)c.pack_bytes + ((double)c.tilenum + 1) * 4.0 : (double)c.tilenum * c.BM * c.BN * vsz);
    }
    return TSP_OK;
}

extern "C" int tsp_time(tsp_handle *h, int cls, const void *d_b, float *d_c, int colB, int iters, float *ms)
{
    if (!h || !d_b || !d_c || !ms || iters <= 0 || cls > 2) { tsp_set_error("time: bad argument"); return TSP_EINVAL; }
    if (!h->converted) { tsp_set_error("time: convert first"); return TSP_ESTATE; }
    TSP_TRY(check_width(colB));
    TSP_CUDA(cudaSetDevice(h->device));
    TSP_TRY(ensure_schedules(h, colB));
    cudaStream_t s = 0;
    TSP_CUDA(cudaEventRecord(h->t0, s));
    for (int i = 0; i < iters; i++)
    {
        if (cls < 0) TSP_TRY(spmm_on(h, d_b, d_c, colB, s));
        else if (h->cls[cls].ntasks > 0) TSP_TRY(launch_class(h, cls, d_b, d_c, colB, s));
    }
    TSP_CUDA(cudaEventRecord(h->t1, s));
    TSP_CUDA(cudaEventSynchronize(h->t1));
    float total = 0.f;
    TSP_CUDA(cudaEventElapsedTime(&total, h->t0, h->t1));
    *ms = total / iters;
    return check_device_error(h);
}

// upstream src/csr2tile.h:906-1019: candidate thresholds per class, then every combination timed on the GPU
extern "C" int tsp_tune(tsp_handle *h, const void *d_b, float *d_c, int colB, int *best3, float *tune_ms)
{
    if (!h || !d_b || !d_c || !best3) { tsp_set_error("tune: null argument"); return TSP_EINVAL; }
    if (!h->converted) { tsp_set_error("tune: convert first"); return TSP_ESTATE; }
    TSP_TRY(check_width(colB));
    TSP_CUDA(cudaSetDevice(h->device));
    int cand[3][4], ncand[3];
    for (int k = 0; k < 3; k++)
    {
        int top4[4] = {32, 32, 32, 32};
        if (h->cls[k].tilenum > 0) TSP_TRY(tsp_top4(h, k, colB, top4));
        ncand[k] = 0;
        const int opts = h->cls[k].tilenum > 0 ? 4 : 1;
        for (int i = 0; i < opts; i++)  // de-duplicate, keeping order (src/csr2tile.h:921-941)
        {
            bool dup = false;
            for (int j = 0; j < ncand[k]; j++) if (cand[k][j] == top4[i]) dup = true;
            if (!dup) cand[k][ncand[k]++] = top4[i];
        }
        best3[k] = cand[k][0];
        if (h->cls[k].tilem > 0) TSP_TRY(tsp_schedule(h, k, cand[k][0]));
    }
    cudaStream_t s = 0;
    cudaEvent_t a, b;
    TSP_CUDA(cudaEventCreate(&a));
    TSP_CUDA(cudaEventCreate(&b));
    TSP_CUDA(cudaEventRecord(a, s));
    float best_ms = 1e12f;
    if (ncand[0] * ncand[1] * ncand[2] > 1)
    {
        for (int i = 0; i < ncand[0]; i++)
            for (int j = 0; j < ncand[1]; j++)
                for (int k = 0; k < ncand[2]; k++)
                {
                    const int th[3] = {cand[0][i], cand[1][j], cand[2][k]};
                    for (int q = 0; q < 3; q++)
                        if (h->cls[q].tilem > 0 && h->cls[q].TH != th[q]) TSP_TRY(tsp_schedule(h, q, th[q]));
                    for (int w = 0; w < 5; w++) TSP_TRY(spmm_on(h, d_b, d_c, colB, s));
                    TSP_CUDA(cudaEventRecord(h->t0, s));
                    for (int w = 0; w < 10; w++) TSP_TRY(spmm_on(h, d_b, d_c, colB, s));
                    TSP_CUDA(cudaEventRecord(h->t1, s));
                    TSP_CUDA(cudaEventSynchronize(h->t1));
                    float ms = 0.f;
                    TSP_CUDA(cudaEventElapsedTime(&ms, h->t0, h->t1));
                    if (ms < best_ms) { best_ms = ms; best3[0] = th[0]; best3[1] = th[1]; best3[2] = th[2]; }
                }
        for (int q = 0; q < 3; q++)
            if (h->cls[q].tilem > 0 && h->cls[q].TH != best3[q]) TSP_TRY(tsp_schedule(h, q, best3[q]));
    }
    TSP_CUDA(cudaEventRecord(b, s));
    TSP_CUDA(cudaEventSynchronize(b));
    float total = 0.f;
    TSP_CUDA(cudaEventElapsedTime(&total, a, b));
    cudaEventDestroy(a); cudaEventDestroy(b);
    if (tune_ms) *tune_ms = total;
    return check_device_error(h);
}

// SM clock in MHz through NVML (read only), or 0 when NVML is not available -- upstream get_gpu_clock (src/common.h:96-119)
static unsigned int sm_clock_mhz(int device)
{
    typedef int (*InitFn)(void);
    typedef int (*FindFn)(const char *, void **);
    typedef int (*ClockFn)(void *, unsigned int, unsigned int *);
    static void *dev[64];
    static ClockFn clock_fn = nullptr;
    static bool tried = false;
    static FindFn find_fn = nullptr;
    if (!tried)
    {
        tried = true;
        void *lib = dlopen("libnvidia-ml.so.1", RTLD_LAZY);
        InitFn init = lib ? (InitFn)dlsym(lib, "nvmlInit_v2") : nullptr;
        find_fn = lib ? (FindFn)dlsym(lib, "nvmlDeviceGetHandleByPciBusId_v2") : nullptr;
        clock_fn = lib ? (ClockFn)dlsym(lib, "nvmlDeviceGetClockInfo") : nullptr;
        if (!init || !find_fn || !clock_fn || init() != 0) clock_fn = nullptr;
    }
    if (!clock_fn || device < 0 || device >= 64) return 0;
    if (!dev[device])
    {
        char pci[32];
        if (cudaDeviceGetPCIBusId(pci, sizeof(pci), device) != cudaSuccess || find_fn(pci, &dev[device]) != 0) { dev[device] = nullptr; return 0; }
    }
    unsigned int mhz = 0;
    return clock_fn(dev[device], 1 /* NVML_CLOCK_SM */, &mhz) == 0 ? mhz : 0;
}

// Warm-up with clock stabilisation, upstream warmup_gpu (src/csr2tile.h:798-823): 20 passes, then batches of 50 until two
// consecutive SM clock readings are at least 95% of the device clock rate and within 2% of each other; at most 1000
// passes, or a fixed 100 when the clock cannot be read.
static int warmup_like_upstream(tsp_handle *h, const void *d_b, float *d_c, int colB)
{
    int reference_khz = 0;
    cudaDeviceGetAttribute(&reference_khz, cudaDevAttrClockRate, h->device);
    const int limit = reference_khz > 0 && sm_clock_mhz(h->device) ? 1000 : 100;
    unsigned int previous = 0;
    for (int total = 0; total < limit;)
    {
        int count = total == 0 ? 20 : 50;
        if (count > limit - total) count = limit - total;
        for (int i = 0; i < count; i++) TSP_TRY(spmm_on(h, d_b, d_c, colB, 0));
        TSP_CUDA(cudaStreamSynchronize(0));
        total += count;
        const unsigned int current = sm_clock_mhz(h->device);
        if (reference_khz > 0 && previous && current && previous * 1000.0 >= reference_khz * 0.95 && current * 1000.0 >= reference_khz * 0.95 &&
            fabsf((float)current / previous - 1.0f) <= 0.02f)
            break;
        previous = current;
    }
    return TSP_OK;
}

static double now_ms()
{
    struct timeval t;
    gettimeofday(&t, nullptr);
    return t.tv_sec * 1000.0 + t.tv_usec / 1000.0;
}

extern "C" int tsp_run(tsp_handle *h, const void *h_b, float *h_c, int colB, int colB_logical, double cpu_pre_ms, int repeat, double *out6)
{
    if (!h || !h_b || !out6 || repeat <= 0) { tsp_set_error("run: bad argument"); return TSP_EINVAL; }
    if (!h->converted) { tsp_set_error("run: convert first"); return TSP_ESTATE; }
    TSP_TRY(check_width(colB));
    TSP_CUDA(cudaSetDevice(h->device));
    const size_t vsz = h->precision ? 4 : 2;
    const size_t b_bytes = (size_t)h->colA * colB * vsz, c_bytes = (size_t)tsp_c_rows(h) * colB * 4;
    void *d_b = nullptr;
    float *d_c = nullptr;
    TSP_CUDA(cudaMalloc(&d_b, b_bytes));
    cudaError_t e = cudaMalloc((void **)&d_c, c_bytes);
    if (e != cudaSuccess) { cudaFree(d_b); tsp_set_error("run: cudaMalloc C: %s", cudaGetErrorString(e)); return TSP_ENOMEM; }
    int rc = TSP_OK;
    auto bail = [&](int code) { cudaFree(d_b); cudaFree(d_c); return code; };
    if (cudaMemcpy(d_b, h_b, b_bytes, cudaMemcpyHostToDevice) != cudaSuccess || cudaMemset(d_c, 0, c_bytes) != cudaSuccess)
    {
        tsp_set_error("run: upload failed");
        return bail(TSP_ECUDA);
    }
    // threshold candidates (host cost model) + tuning, both counted as preprocessing like upstream (src/csr2tile.h:1061)
    const double t_a = now_ms();
    for (int k = 0; k < 3; k++) h->cls[k].TH = 0;
    if ((rc = ensure_schedules(h, colB)) != TSP_OK) return bail(rc);
    const double cand_ms = now_ms() - t_a;
    if ((rc = warmup_like_upstream(h, d_b, d_c, colB)) != TSP_OK) return bail(rc);
    int best3[3];
    float tune_ms = 0.f;
    if ((rc = tsp_tune(h, d_b, d_c, colB, best3, &tune_ms)) != TSP_OK) return bail(rc);
    if ((rc = spmm_on(h, d_b, d_c, colB, 0)) != TSP_OK) return bail(rc);
    if (cudaDeviceSynchronize() != cudaSuccess) { tsp_set_error("run: checked pass failed: %s", cudaGetErrorString(cudaGetLastError())); return bail(TSP_ECUDA); }
    if ((rc = check_device_error(h)) != TSP_OK) return bail(rc);
    if (h_c && cudaMemcpy(h_c, d_c, (size_t)(h->row_end - h->row_begin) * colB * 4, cudaMemcpyDeviceToHost) != cudaSuccess)
    {
        tsp_set_error("run: copy of C failed");
        return bail(TSP_ECUDA);
    }
    if ((rc = warmup_like_upstream(h, d_b, d_c, colB)) != TSP_OK) return bail(rc);
    float ms = 0.f;
    if ((rc = tsp_time(h, -1, d_b, d_c, colB, repeat, &ms)) != TSP_OK) return bail(rc);
    out6[0] = best3[0]; out6[1] = best3[1]; out6[2] = best3[2];
    out6[3] = cpu_pre_ms + cand_ms + tune_ms;
    out6[4] = ms;
    out6[5] = (2.0 * (double)h->nnzA * 1.0e-6 / ms * colB_logical) / 1000.0;  // src/csr2tile.h:1057
    return bail(TSP_OK);
}

// upstream cusparse_spmm_all (src/main.cu:16-134)
static int cusparse_baseline(int device, int precision, int m, int k, long long nnz, const int *rp, const int *ci, const void *val,
                             int n, int ldb, const void *h_b, float *h_c, int warmup, int repeat, int alg_id, double *out3);

extern "C" int tsp_cusparse_baseline(int device, int precision, int m, int k, long long nnz, const int *rp, const int *ci, const void *val,
                                     int n, int ldb, const void *h_b, float *h_c, int warmup, int repeat, double *out3)
{
    return cusparse_baseline(device, precision, m, k, nnz, rp, ci, val, n, ldb, h_b, h_c, warmup, repeat, 0, out3);
}

extern "C" int tsp_cusparse_baseline_alg(int device, int precision, int m, int k, long long nnz, const int *rp, const int *ci, const void *val,
                                         int n, int ldb, const void *h_b, float *h_c, int warmup, int repeat, int alg, double *out3)
{
    if (alg < 0 || alg > 3) { tsp_set_error("cusparse_baseline_alg: alg must be 0 (default), 1, 2 or 3 (CSR_ALG1..3)"); return TSP_EINVAL; }
    return cusparse_baseline(device, precision, m, k, nnz, rp, ci, val, n, ldb, h_b, h_c, warmup, repeat, alg, out3);
}

static int cusparse_baseline(int device, int precision, int m, int k, long long nnz, const int *rp, const int *ci, const void *val,
                             int n, int ldb, const void *h_b, float *h_c, int warmup, int repeat, int alg_id, double *out3)
{
    if (!rp || !ci || !val || !h_b || !out3 || repeat <= 0) { tsp_set_error("cusparse_baseline: bad argument"); return TSP_EINVAL; }
    const cusparseSpMMAlg_t alg = alg_id == 1 ? CUSPARSE_SPMM_CSR_ALG1 : alg_id == 2 ? CUSPARSE_SPMM_CSR_ALG2 : alg_id == 3 ? CUSPARSE_SPMM_CSR_ALG3 : CUSPARSE_SPMM_ALG_DEFAULT;
    TSP_CUDA(cudaSetDevice(device));
    const size_t vsz = precision ? 4 : 2;
    int *d_rp = nullptr, *d_ci = nullptr;
    void *d_v = nullptr, *d_b = nullptr, *buf = nullptr;
    float *d_c = nullptr;
    cusparseHandle_t handle = nullptr;
    cusparseSpMatDescr_t A = nullptr;
    cusparseDnMatDescr_t B = nullptr, Cm = nullptr;
    cudaEvent_t t0 = nullptr, t1 = nullptr;
    int rc = TSP_OK;
    auto fail = [&](const char *what) { tsp_set_error("cusparse_baseline: %s failed", what); rc = TSP_ECUDA; };
    do
    {
        if (cudaMalloc((void **)&d_rp, ((size_t)m + 1) * 4) || cudaMalloc((void **)&d_ci, (size_t)nnz * 4) || cudaMalloc(&d_v, (size_t)nnz * vsz) ||
            cudaMalloc(&d_b, (size_t)k * ldb * vsz) || cudaMalloc((void **)&d_c, (size_t)m * n * 4)) { fail("cudaMalloc"); break; }
        if (cudaMemcpy(d_rp, rp, ((size_t)m + 1) * 4, cudaMemcpyHostToDevice) || cudaMemcpy(d_ci, ci, (size_t)nnz * 4, cudaMemcpyHostToDevice) ||
            cudaMemcpy(d_v, val, (size_t)nnz * vsz, cudaMemcpyHostToDevice) || cudaMemcpy(d_b, h_b, (size_t)k * ldb * vsz, cudaMemcpyHostToDevice) ||
            cudaMemset(d_c, 0, (size_t)m * n * 4)) { fail("upload"); break; }
        const double t_a = now_ms();
        const cudaDataType vt = precision ? CUDA_R_32F : CUDA_R_16F;  // true FP32 for the TF32 build (src/main.cu:54-63)
        if (cusparseCreate(&handle) || cusparseSetStream(handle, cudaStreamLegacy)) { fail("cusparseCreate"); break; }
        if (cusparseCreateCsr(&A, m, k, nnz, d_rp, d_ci, d_v, CUSPARSE_INDEX_32I, CUSPARSE_INDEX_32I, CUSPARSE_INDEX_BASE_ZERO, vt) ||
            cusparseCreateDnMat(&B, k, n, ldb, d_b, vt, CUSPARSE_ORDER_ROW) || cusparseCreateDnMat(&Cm, m, n, n, d_c, CUDA_R_32F, CUSPARSE_ORDER_ROW))
        { fail("descriptor creation"); break; }
        const float alpha = 1.0f, beta = 0.0f;
        size_t bytes = 0;
        if (cusparseSpMM_bufferSize(handle, CUSPARSE_OPERATION_NON_TRANSPOSE, CUSPARSE_OPERATION_NON_TRANSPOSE, &alpha, A, B, &beta, Cm, CUDA_R_32F,
                                    alg, &bytes)) { fail("cusparseSpMM_bufferSize"); break; }
        if (cudaMalloc(&buf, bytes ? bytes : 1)) { fail("cudaMalloc buffer"); break; }
        // the non-default algorithms may analyse the matrix once; that time goes into pre_time like every other set-up step
        if (alg_id != 0 && cusparseSpMM_preprocess(handle, CUSPARSE_OPERATION_NON_TRANSPOSE, CUSPARSE_OPERATION_NON_TRANSPOSE, &alpha, A, B, &beta, Cm,
                                                   CUDA_R_32F, alg, buf)) { fail("cusparseSpMM_preprocess"); break; }
        if (cudaDeviceSynchronize()) { fail("cusparseSpMM_preprocess"); break; }
        out3[0] = now_ms() - t_a;
        bool bad = false;
        for (int i = 0; i < warmup && !bad; i++)
            bad = cusparseSpMM(handle, CUSPARSE_OPERATION_NON_TRANSPOSE, CUSPARSE_OPERATION_NON_TRANSPOSE, &alpha, A, B, &beta, Cm, CUDA_R_32F,
                               alg, buf) != CUSPARSE_STATUS_SUCCESS;
        if (bad || cudaDeviceSynchronize()) { fail("cusparseSpMM warm-up"); break; }
        cudaEventCreate(&t0); cudaEventCreate(&t1);
        cudaEventRecord(t0, cudaStreamLegacy);
        for (int i = 0; i < repeat && !bad; i++)
            bad = cusparseSpMM(handle, CUSPARSE_OPERATION_NON_TRANSPOSE, CUSPARSE_OPERATION_NON_TRANSPOSE, &alpha, A, B, &beta, Cm, CUDA_R_32F,
                               alg, buf) != CUSPARSE_STATUS_SUCCESS;
        cudaEventRecord(t1, cudaStreamLegacy);
        if (bad || cudaEventSynchronize(t1)) { fail("cusparseSpMM"); break; }
        float ms = 0.f;
        cudaEventElapsedTime(&ms, t0, t1);
        out3[1] = ms / repeat;
        out3[2] = (2.0 * (double)nnz * (double)n / (out3[1] / 1000.0)) / 1e12;
        if (h_c && cudaMemcpy(h_c, d_c, (size_t)m * n * 4, cudaMemcpyDeviceToHost)) { fail("copy of C"); break; }
    } while (0);
    if (t0) cudaEventDestroy(t0);
    if (t1) cudaEventDestroy(t1);
    if (B) cusparseDestroyDnMat(B);
    if (Cm) cusparseDestroyDnMat(Cm);
    if (A) cusparseDestroySpMat(A);
    if (handle) cusparseDestroy(handle);
    cudaFree(buf); cudaFree(d_rp); cudaFree(d_ci); cudaFree(d_v); cudaFree(d_b); cudaFree(d_c);
    return rc;
}
