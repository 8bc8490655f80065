// Load balancing: threshold candidates from the cost model and the task arrays for one threshold.
//
// Replaces upstream get_optimal_prefetch_th (src/csr2tile.h:437-642), tile_pretreatment (src/csr2tile.h:383-434)
// and update_metadata (src/csr2tile.h:644-711).  The task arrays are built on the device from tile_ptr
// (upstream: host loop + upload per tuning combination); the cost model runs on the host over the histogram
// of tiles per panel, in float and in upstream's evaluation order, with the resource rows of THESE kernels.
#include <cub/cub.cuh>
#include <math.h>
#include <stdlib.h>

#include <mutex>

#include "tsp_internal.cuh"

void tsp_small_resources(int precision, int cls, int colB, TspKernelResources *out);
void tsp_class64_resources(int precision, int colB, TspKernelResources *out);

void tsp_kernel_resources(int precision, int cls, int colB, TspKernelResources *out)
{
    if (cls == 0) tsp_class64_resources(precision, colB, out);
    else tsp_small_resources(precision, cls, colB, out);
}

namespace
{

__global__ void k_task_counts(int tilem, const int *__restrict__ tile_ptr, int TH, int *__restrict__ counts)
{
    int p = blockIdx.x * blockDim.x + threadIdx.x;
    if (p > tilem) return;
    if (p == tilem) { counts[p] = 0; return; }
    const int len = tile_ptr[p + 1] - tile_ptr[p];
    counts[p] = len <= TH ? 1 : (len + TH - 1) / TH;  // src/csr2tile.h:392-396
}

__global__ void k_task_fill(int tilem, const int *__restrict__ tile_ptr, const int *__restrict__ panel_row, int TH,
                            const int *__restrict__ task_base, unsigned int *__restrict__ task_row, int *__restrict__ task_start,
                            int *__restrict__ split_row, int *__restrict__ split_count)
{
    int p = blockIdx.x * blockDim.x + threadIdx.x;
    if (p >= tilem) return;
    const int t0 = tile_ptr[p], len = tile_ptr[p + 1] - t0, b = task_base[p], row = panel_row[p];
    if (p == 0) task_start[0] = t0;
    if (len <= TH)
    {
        task_row[b] = (unsigned int)row;
        task_start[b + 1] = t0 + len;
        return;
    }
    const int parts = (len + TH - 1) / TH, each = (len + parts - 1) / parts;  // src/csr2tile.h:421-422
    for (int s = 0; s < parts; s++)
    {
        task_row[b + s] = (unsigned int)row | 0x80000000u;
        task_start[b + s + 1] = s == parts - 1 ? t0 + len : t0 + (s + 1) * each;
    }
    split_row[atomicAdd(split_count, 1)] = row;
}

// sort key of a task: longer tasks get smaller keys
__global__ void k_task_keys(int ntasks, const int *__restrict__ task_start, unsigned int *__restrict__ keys, int *__restrict__ ids)
{
    int t = blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= ntasks) return;
    const int len = task_start[t + 1] - task_start[t];
    keys[t] = 0xffffu - (unsigned int)(len > 0xffff ? 0xffff : len);
    ids[t] = t;
}

__global__ void k_task_pack(int ntasks, const int *__restrict__ order, const unsigned int *__restrict__ task_row,
                            const int *__restrict__ task_start, uint4 *__restrict__ pack)
{
    int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= ntasks) return;
    const int t = order ? order[i] : i;
    pack[i] = make_uint4(task_row[t], (unsigned int)task_start[t], (unsigned int)task_start[t + 1], 0u);
}

// The 16/8-row kernels run four tasks per CTA, one per warp, and a CTA holds its SM resources until its longest
// task is done.  Walking the tasks longest first (stable, so equal tasks keep their panel order and with it the
// locality of their B rows in L2) puts tasks of similar length into one CTA and the long ones at the front of the
// launch.  TSP_TASK_ORDER=0 in the environment keeps panel order.
int build_task_pack(TspClass &c)
{
    if (c.ntasks == 0) return TSP_OK;
    static int sorted = -1;
    if (sorted < 0) { const char *e = getenv("TSP_TASK_ORDER"); sorted = (e && e[0] == '0') ? 0 : 1; }
    const int T = 256, n = c.ntasks;
    unsigned int *keys = nullptr, *keys_out = nullptr;
    int *ids = nullptr, *ids_out = nullptr;
    void *scratch = nullptr;
    cudaError_t e = cudaSuccess;
    if (sorted)
    {
        size_t bytes = 0;
        e = cudaMalloc((void **)&keys, (size_t)n * 16);   // keys, sorted keys, ids, sorted ids
        if (e == cudaSuccess)
        {
            keys_out = keys + n; ids = (int *)(keys + 2 * (size_t)n); ids_out = ids + n;
            k_task_keys<<<(n + T - 1) / T, T>>>(n, c.d_task_start, keys, ids);
            e = cub::DeviceRadixSort::SortPairs(nullptr, bytes, keys, keys_out, ids, ids_out, n, 0, 16);
        }
        if (e == cudaSuccess) e = cudaMalloc(&scratch, bytes ? bytes : 1);
        if (e == cudaSuccess) e = cub::DeviceRadixSort::SortPairs(scratch, bytes, keys, keys_out, ids, ids_out, n, 0, 16);
    }
    if (e == cudaSuccess)
    {
        k_task_pack<<<(n + T - 1) / T, T>>>(n, sorted ? ids_out : nullptr, c.d_task_row, c.d_task_start, c.d_task_pack);
        e = cudaGetLastError();
    }
    if (e == cudaSuccess) e = cudaDeviceSynchronize();   // the scratch goes away below
    cudaFree(scratch); cudaFree(keys);
    TSP_CUDA(e);
    return TSP_OK;
}

}  // namespace

int tsp_schedule(tsp_handle *h, int cls, int TH)
{
    if (!h || cls < 0 || cls > 2 || TH <= 0) { tsp_set_error("schedule: bad argument"); return TSP_EINVAL; }
    if (!h->converted) { tsp_set_error("schedule: convert first"); return TSP_ESTATE; }
    TSP_CUDA(cudaSetDevice(h->device));
    TspRange range("tsp schedule");
    TspClass &c = h->cls[cls];
    c.TH = TH; c.ntasks = 0; c.nsplit = 0;
    if (c.tilem == 0) return TSP_OK;
    if (!c.d_task_count || c.tilem > c.cap_panels)
    {
        cudaFree(c.d_task_count); cudaFree(c.d_split_row);
        c.d_task_count = nullptr; c.d_split_row = nullptr; c.cap_panels = 0;
        TSP_CUDA(cudaMalloc((void **)&c.d_task_count, ((size_t)c.tilem + 2) * 4));
        TSP_CUDA(cudaMalloc((void **)&c.d_split_row, ((size_t)c.tilem + 1) * 4));
        c.cap_panels = c.tilem;
    }
    const int T = 256;
    k_task_counts<<<(c.tilem + 1 + T - 1) / T, T>>>(c.tilem, c.d_tile_ptr, TH, c.d_task_count);
    TSP_CUDA(cudaGetLastError());
    size_t bytes = 0;
    TSP_CUDA(cub::DeviceScan::ExclusiveSum(nullptr, bytes, c.d_task_count, c.d_task_count, c.tilem + 1));
    void *scratch = nullptr;
    TSP_CUDA(cudaMalloc(&scratch, bytes ? bytes : 1));
    cudaError_t e = cub::DeviceScan::ExclusiveSum(scratch, bytes, c.d_task_count, c.d_task_count, c.tilem + 1);
    int ntasks = 0;
    if (e == cudaSuccess) e = cudaMemcpy(&ntasks, c.d_task_count + c.tilem, 4, cudaMemcpyDeviceToHost);
    cudaFree(scratch);
    TSP_CUDA(e);
    if ((long long)ntasks > c.cap_tasks)
    {
        cudaFree(c.d_task_row); cudaFree(c.d_task_start); cudaFree(c.d_task_pack);
        c.d_task_row = nullptr; c.d_task_start = nullptr; c.d_task_pack = nullptr;
        c.cap_tasks = (long long)ntasks + ntasks / 4 + 16;
        TSP_CUDA(cudaMalloc((void **)&c.d_task_row, (size_t)c.cap_tasks * 4));
        TSP_CUDA(cudaMalloc((void **)&c.d_task_start, ((size_t)c.cap_tasks + 1) * 4));
        if (cls != 0) TSP_CUDA(cudaMalloc((void **)&c.d_task_pack, (size_t)c.cap_tasks * sizeof(uint4)));
    }
    int *d_split_count = c.d_task_count + c.tilem + 1;
    TSP_CUDA(cudaMemset(d_split_count, 0, 4));
    k_task_fill<<<(c.tilem + T - 1) / T, T>>>(c.tilem, c.d_tile_ptr, c.d_panel_row, TH, c.d_task_count, c.d_task_row, c.d_task_start,
                                             c.d_split_row, d_split_count);
    TSP_CUDA(cudaGetLastError());
    TSP_CUDA(cudaMemcpy(&c.nsplit, d_split_count, 4, cudaMemcpyDeviceToHost));
    c.ntasks = ntasks;
    if (cls != 0) TSP_TRY(build_task_pack(c));
    return TSP_OK;
}

int tsp_export_schedule(const tsp_handle *h, int cls, int *ntasks, unsigned int *h_rows, int *h_colstart)
{
    if (!h || cls < 0 || cls > 2 || !ntasks) { tsp_set_error("export_schedule: bad argument"); return TSP_EINVAL; }
    const TspClass &c = h->cls[cls];
    *ntasks = c.ntasks;
    if (c.ntasks == 0) return TSP_OK;
    if (h_rows) TSP_CUDA(cudaMemcpy(h_rows, c.d_task_row, (size_t)c.ntasks * 4, cudaMemcpyDeviceToHost));
    if (h_colstart) TSP_CUDA(cudaMemcpy(h_colstart, c.d_task_start, ((size_t)c.ntasks + 1) * 4, cudaMemcpyDeviceToHost));
    return TSP_OK;
}

#include "atom_table.inc"

// Weight of one atomic slice in the cost model below: upstream's table has this shape (one row for 32 columns, one for
// wider right-hand sides, src/csr2tile.h:483-495) but holds constants fitted to its kernels on its GPUs; the values
// here are fitted to these kernels on B200 by tilespmm_b200/calibrate_atom.py.
float tsp_atom_weight(int precision, int cls, int colB_padded)
{
    if (cls < 0 || cls > 2) return 0.01f;
    return kAtomWeight[colB_padded == 32 ? 0 : 1][cls][precision ? 1 : 0];
}

// The four cheapest thresholds under the upstream cost model (src/csr2tile.h:437-642).
int tsp_top4(const tsp_handle *h, int cls, int colB, int *top4)
{
    if (!h || cls < 0 || cls > 2 || !top4 || colB <= 0) { tsp_set_error("top4: bad argument"); return TSP_EINVAL; }
    if (!h->converted) { tsp_set_error("top4: convert first"); return TSP_ESTATE; }
    for (int i = 0; i < 4; i++) top4[i] = 32;
    const TspClass &c = h->cls[cls];
    if (c.tilenum == 0) return TSP_OK;
    TspKernelResources R;
    tsp_kernel_resources(h->precision, cls, colB, &R);
    const int is_tf32 = h->precision, BM = c.BM;
    const int sm = h->prop.multiProcessorCount;
    int blk_reg = h->prop.regsPerMultiprocessor / (R.registers_per_thread > 0 ? R.registers_per_thread * R.threads : 1);
    int blk_smem = R.shared_bytes > 0 ? (int)(h->prop.sharedMemPerMultiprocessor / (size_t)R.shared_bytes) : h->prop.maxBlocksPerMultiProcessor;
    int blk_sm = h->prop.maxThreadsPerMultiProcessor / R.threads;
    if (blk_reg < blk_sm) blk_sm = blk_reg;
    if (blk_smem < blk_sm) blk_sm = blk_smem;
    if (blk_sm > h->prop.maxBlocksPerMultiProcessor) blk_sm = h->prop.maxBlocksPerMultiProcessor;
    if (blk_sm <= 0) { tsp_set_error("top4: the kernel does not fit this GPU"); return TSP_EDEVICE; }
    const float cap = (float)(blk_sm * sm);
    const float lambda_l2 = (float)(R.iteration_bytes * cap) / (float)h->prop.l2CacheSize;
    const float lambda_atom = tsp_atom_weight(is_tf32, cls, colB);
    const float atom_per_col = lambda_atom * (1.0f / 32.0f);

    const std::vector<int> &tp = c.h_tile_ptr;
    int max_len = 0;
    long long total_len = 0;
    for (int p = 0; p < c.tilem; p++)
    {
        const int len = tp[p + 1] - tp[p];
        if (len > max_len) max_len = len;
        total_len += len;
    }
    if (max_len == 0) return TSP_OK;
    std::vector<int> hist((size_t)max_len + 1, 0);
    for (int p = 0; p < c.tilem; p++) hist[tp[p + 1] - tp[p]]++;
    hist[0] = 0;
    std::vector<int> lens;
    for (int len = 1; len <= max_len; len++) if (hist[len]) lens.push_back(len);

    const float avg_len = (float)total_len / c.tilem;
    float atom_pen = atom_per_col * (float)colB;
    if (max_len > avg_len * 5.0f) atom_pen *= 0.04f;
    int tmax = (max_len + 7) / 8 * 8;
    if (tmax > 128) tmax = 128;
    // one block of these kernels serves tasks_per_block tasks of one stripe
    const int stripe = tsp_stripe_width(cls, colB);
    int cand_th[16], ncand = 0;
    float cand_cost[16];
    long long prev_tasks = -1;
    for (int TH = 8; TH <= tmax; TH += 8)
    {
        long long atom_ops = 0, tasks = 0;
        int max_chunk = 0;
        float l2_penalty = 0.0f;
        for (int len : lens)
        {
            const int cnt = hist[len];
            const int parts = (len + TH - 1) / TH, each = (len + parts - 1) / parts;
            atom_ops += (long long)(parts - 1) * cnt;
            tasks += (long long)parts * cnt;
            if (each > max_chunk) max_chunk = each;
            if (parts > 1) l2_penalty += (1.0f - (1.0f / (float)parts)) * cnt;
        }
        if (tasks == prev_tasks) continue;
        prev_tasks = tasks;
        const long long blocks = (tasks * (colB / stripe) + R.tasks_per_block - 1) / R.tasks_per_block;
        const float cost_base = (float)blocks / cap * TH;
        const float cost_tail = (float)max_chunk;
        const float cost_l2 = l2_penalty * lambda_l2;
        const float cost_comp = cost_base + cost_tail + cost_l2;
        const float cost_atom = atom_pen * atom_ops;
        cand_th[ncand] = TH;
        cand_cost[ncand] = cost_comp + cost_atom;
        ncand++;
    }
    for (int i = 1; i < ncand; i++)  // stable: ties keep ascending TH (src/csr2tile.h:620-631)
    {
        const int th = cand_th[i];
        const float cost = cand_cost[i];
        int j = i - 1;
        while (j >= 0 && cand_cost[j] > cost) { cand_th[j + 1] = cand_th[j]; cand_cost[j + 1] = cand_cost[j]; j--; }
        cand_th[j + 1] = th; cand_cost[j + 1] = cost;
    }
    for (int i = 0; i < 4; i++) top4[i] = i < ncand ? cand_th[i] : cand_th[0];
    return TSP_OK;
}

// ---------------------------------------------------------------------------------------------------------
// Scheduling without any allocation.
//
// tsp_schedule() above sizes and allocates its per-panel counters and its scan workspace with cudaMalloc.
// Some hosts cannot do that at the point where they need a new schedule: a solver or serving process that
// carves all device memory into its own arena at start-up (so a later cudaMalloc may simply fail, and
// cudaMalloc/cudaFree would stall the whole device on its hot path), or a real-time loop that is not allowed
// to enter the allocator at all.  For them tsp_schedule_noalloc() does the same work with the per-panel
// counters kept in the fixed device array below, which every GPU that loads this library holds until the
// process exits (4 MB + 260 B).  The caller provides the tile pointers, the panel rows and the output arrays.
// ---------------------------------------------------------------------------------------------------------

#define TSP_NOALLOC_MAX_PANELS (1 << 20)

// [0 .. tilem]            per-panel task counts, scanned in place
// [MAX_PANELS + 1 ...]    counter of split panels
static __device__ __align__(256) int g_noalloc_scratch[TSP_NOALLOC_MAX_PANELS + 1 + 64];

namespace
{

// In-place exclusive scan of a[0..n) by ONE block of exactly 1024 threads (all 32 warp_sum slots are written every
// pass); n <= about a million ints: a few passes.
constexpr int SCAN_THREADS = 1024;
__global__ void __launch_bounds__(SCAN_THREADS) k_scan_one_block(int *a, int n)
{
    __shared__ int warp_sum[32];
    __shared__ int carry;
    if (threadIdx.x == 0) carry = 0;
    __syncthreads();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (int base = 0; base < n; base += blockDim.x)
    {
        const int i = base + threadIdx.x;
        const int v = i < n ? a[i] : 0;
        int x = v;
        for (int o = 1; o < 32; o <<= 1) { const int y = __shfl_up_sync(0xffffffffu, x, o); if (lane >= o) x += y; }
        if (lane == 31) warp_sum[warp] = x;
        __syncthreads();
        if (warp == 0)
        {
            int w = warp_sum[lane];
            for (int o = 1; o < 32; o <<= 1) { const int y = __shfl_up_sync(0xffffffffu, w, o); if (lane >= o) w += y; }
            warp_sum[lane] = w;
        }
        __syncthreads();
        const int before = carry + (warp ? warp_sum[warp - 1] : 0) + x - v;
        if (i < n) a[i] = before;
        __syncthreads();
        if (threadIdx.x == blockDim.x - 1) carry = before + v;
        __syncthreads();
    }
}

// Same output as k_task_fill, but never writes past the caller's capacity.
__global__ void k_task_fill_bounded(int tilem, const int *__restrict__ tile_ptr, const int *__restrict__ panel_row, int TH,
                                    const int *__restrict__ task_base, long long capacity, unsigned int *__restrict__ task_row,
                                    int *__restrict__ task_start, int *__restrict__ split_row, int *__restrict__ split_count)
{
    int p = blockIdx.x * blockDim.x + threadIdx.x;
    if (p >= tilem) return;
    if (task_base[tilem] > capacity) return;  // the host reports the overflow; nothing is written
    const int t0 = tile_ptr[p], len = tile_ptr[p + 1] - t0, b = task_base[p], row = panel_row[p];
    if (p == 0) task_start[0] = t0;
    if (len <= TH)
    {
        task_row[b] = (unsigned int)row;
        task_start[b + 1] = t0 + len;
        return;
    }
    const int parts = (len + TH - 1) / TH, each = (len + parts - 1) / parts;
    for (int s = 0; s < parts; s++)
    {
        task_row[b + s] = (unsigned int)row | 0x80000000u;
        task_start[b + s + 1] = s == parts - 1 ? t0 + len : t0 + (s + 1) * each;
    }
    const int slot = atomicAdd(split_count, 1);
    if (split_row) split_row[slot] = row;
}

int *g_noalloc_ptr[64];       // device address of g_noalloc_scratch per device, resolved on first use
bool g_noalloc_ready[64];
std::mutex g_noalloc_mutex;   // two host threads may make their first call on a device at the same time

// restores the caller's current device when the entry point returns
struct DeviceGuard
{
    int previous = -1;
    DeviceGuard() { if (cudaGetDevice(&previous) != cudaSuccess) previous = -1; }
    ~DeviceGuard() { if (previous >= 0) cudaSetDevice(previous); }
};

}  // namespace

// Builds the task arrays of one tile class for threshold TH -- the same arrays tsp_schedule() builds -- without
// calling cudaMalloc, cudaFree or any allocating library routine.
//
//   d_tile_ptr[tilem+1], d_panel_row[tilem]   inputs (device): tiles per panel (prefix sums) and first rows
//   d_task_row[capacity], d_task_start[capacity+1]   outputs (device), caller-allocated
//   d_split_row[tilem]                        output (device, may be NULL): first rows of the split panels
//   *ntasks, *nsplit                          outputs (host)
//
// Limits and rules:
//   * tilem <= TSP_NOALLOC_MAX_PANELS (1,048,576 panels); more is refused with TSP_EINVAL.  If the schedule
//     needs more than `capacity` tasks the call returns TSP_ENOMEM, *ntasks holds the number needed and the
//     output arrays are left untouched.
//   * The first call on a device looks up the device address of the scratch array (with that device current) and, with
//     lazy module loading, is also the call that loads these kernels onto the device -- both may allocate inside the
//     CUDA runtime.  Make that first call at start-up: before any stream capture, and before the host carves its arena.
//     Later calls allocate nothing (the GPU test checks that the free device memory does not move).
//   * All calls share the one scratch array per device.  Each call clears what it needs at its start, so calls
//     one after another on the same stream are fine; two calls whose kernels can overlap on the GPU (different
//     streams or threads, same device) race on it and must be serialised by the caller.
//   * The call waits for `stream` before it returns (it has to read the task count back).
extern "C" int tsp_schedule_noalloc(int device, int tilem, int TH, const int *d_tile_ptr, const int *d_panel_row,
                                    unsigned int *d_task_row, int *d_task_start, long long capacity, int *d_split_row,
                                    int *ntasks, int *nsplit, void *stream)
{
    if (tilem < 0 || TH <= 0 || !d_tile_ptr || !d_panel_row || !d_task_row || !d_task_start || capacity < 0 || !ntasks || device < 0 || device >= 64)
    {
        tsp_set_error("schedule_noalloc: bad argument");
        return TSP_EINVAL;
    }
    if (tilem > TSP_NOALLOC_MAX_PANELS)
    {
        tsp_set_error("schedule_noalloc: %d panels exceed the fixed scratch of %d panels; use tsp_schedule()", tilem, TSP_NOALLOC_MAX_PANELS);
        return TSP_EINVAL;
    }
    DeviceGuard restore_device;
    TSP_CUDA(cudaSetDevice(device));
    {
        std::lock_guard<std::mutex> lock(g_noalloc_mutex);
        if (!g_noalloc_ready[device])
        {
            // In host code the array's name is only a handle for the runtime, not a device address.
            void *p = nullptr;
            TSP_CUDA(cudaGetSymbolAddress(&p, g_noalloc_scratch));
            g_noalloc_ptr[device] = (int *)p;
            g_noalloc_ready[device] = true;
        }
    }
    int *counts = g_noalloc_ptr[device];
    int *split_count = counts + TSP_NOALLOC_MAX_PANELS + 1;
    cudaStream_t s = (cudaStream_t)stream;
    *ntasks = 0;
    if (nsplit) *nsplit = 0;
    if (tilem == 0) return TSP_OK;
    const int T = 256;
    TSP_CUDA(cudaMemsetAsync(split_count, 0, sizeof(int), s));  // the array keeps the previous call's contents
    k_task_counts<<<(tilem + 1 + T - 1) / T, T, 0, s>>>(tilem, d_tile_ptr, TH, counts);
    k_scan_one_block<<<1, SCAN_THREADS, 0, s>>>(counts, tilem + 1);
    k_task_fill_bounded<<<(tilem + T - 1) / T, T, 0, s>>>(tilem, d_tile_ptr, d_panel_row, TH, counts, capacity, d_task_row, d_task_start,
                                                         d_split_row, split_count);
    TSP_CUDA(cudaGetLastError());
    int total = 0, splits = 0;
    TSP_CUDA(cudaMemcpyAsync(&total, counts + tilem, sizeof(int), cudaMemcpyDeviceToHost, s));
    TSP_CUDA(cudaMemcpyAsync(&splits, split_count, sizeof(int), cudaMemcpyDeviceToHost, s));
    TSP_CUDA(cudaStreamSynchronize(s));
    *ntasks = total;
    if ((long long)total > capacity)
    {
        tsp_set_error("schedule_noalloc: the schedule needs %d tasks but the output arrays hold %lld", total, capacity);
        return TSP_ENOMEM;
    }
    if (nsplit) *nsplit = splits;
    return TSP_OK;
}
