// Multi-GPU execution inside ONE process: the panel sequence of a matrix is cut across the GPUs of a box, every GPU
// converts and multiplies its own range and owns the matching row slab of C.
//
// Upstream runs on one GPU only (`-d <device_id>`, src/main.cu:138-142, 210); there is nothing to restate.  The shape
// of this layer follows the single-GPU entry points it wraps: create / convert_host / info / spmm_host / run / destroy,
// with one tsp_handle per device underneath.
//   * conversion: one host thread per device calls tsp_convert_host with that device's shard index; the partition is
//     global and deterministic, so the shards agree with the unsharded tiling.
//   * B: every device uploads only its 1/N row block from host memory, then the blocks are all-gathered over NCCL
//     (NVLink / NVSwitch) into every device's own copy of B, so host-to-device traffic per product does not grow with N
//     and the kernels only ever read local memory -- no peer loads, no multicast loads.
//   * C: row-partitioned, no reduction; every device writes its slab and the slabs are copied back to their rows of
//     the host matrix.
// NCCL is loaded at run time (dlopen), so the library itself has no link-time dependency on it; a process that already
// holds an NCCL (PyTorch's) gets that one.  With one device no collective runs and NCCL is not needed.
#include <dlfcn.h>
#include <stdlib.h>
#include <string.h>
#include <sys/time.h>

#include <thread>

#include "tsp_internal.cuh"

namespace
{

// the few NCCL entry points used here, resolved with dlsym (signatures of nccl.h 2.x)
typedef struct ncclComm *ncclComm_t;
typedef int (*CommInitAllFn)(ncclComm_t *, int, const int *);
typedef int (*CommDestroyFn)(ncclComm_t);
typedef int (*GroupFn)(void);
typedef int (*AllGatherFn)(const void *, void *, size_t, int /* ncclDataType_t */, ncclComm_t, cudaStream_t);
typedef const char *(*ErrorStringFn)(int);
constexpr int kNcclUint8 = 1;   // ncclUint8: the all-gather moves bytes

struct Nccl
{
    void *lib = nullptr;
    CommInitAllFn comm_init_all = nullptr;
    CommDestroyFn comm_destroy = nullptr;
    GroupFn group_start = nullptr, group_end = nullptr;
    AllGatherFn all_gather = nullptr;
    ErrorStringFn error_string = nullptr;
};

int load_nccl(Nccl *n)
{
    const char *names[] = {getenv("TSP_NCCL_LIB"), "libnccl.so.2", "libnccl.so"};
    for (const char *name : names)
    {
        if (!name || !*name) continue;
        n->lib = dlopen(name, RTLD_NOW | RTLD_LOCAL);
        if (n->lib) break;
    }
    if (!n->lib) { tsp_set_error("multi: cannot load NCCL (libnccl.so.2; set TSP_NCCL_LIB to its path): %s", dlerror()); return TSP_ECUDA; }
    n->comm_init_all = (CommInitAllFn)dlsym(n->lib, "ncclCommInitAll");
    n->comm_destroy = (CommDestroyFn)dlsym(n->lib, "ncclCommDestroy");
    n->group_start = (GroupFn)dlsym(n->lib, "ncclGroupStart");
    n->group_end = (GroupFn)dlsym(n->lib, "ncclGroupEnd");
    n->all_gather = (AllGatherFn)dlsym(n->lib, "ncclAllGather");
    n->error_string = (ErrorStringFn)dlsym(n->lib, "ncclGetErrorString");
    if (!n->comm_init_all || !n->comm_destroy || !n->group_start || !n->group_end || !n->all_gather)
    {
        tsp_set_error("multi: the NCCL library lacks an entry point this layer needs");
        return TSP_ECUDA;
    }
    return TSP_OK;
}

double now_ms()
{
    struct timeval t;
    gettimeofday(&t, nullptr);
    return t.tv_sec * 1000.0 + t.tv_usec / 1000.0;
}

}  // namespace

struct tsp_multi
{
    int ndev = 0, precision = 0;
    std::vector<int> dev;
    std::vector<tsp_handle *> h;
    int rowA = 0, colA = 0;
    long long nnz = 0;
    bool converted = false;
    Nccl nccl;
    std::vector<ncclComm_t> comm;
    // per device: its copy of B (block rows * ndev rows), its C slab, one stream
    std::vector<void *> d_b;
    std::vector<float *> d_c;
    std::vector<size_t> b_bytes, c_bytes;
    std::vector<cudaStream_t> stream;
};

#define NCCL_TRY(m, call)                                                                                                 \
    do {                                                                                                                  \
        const int r__ = (call);                                                                                           \
        if (r__ != 0) { tsp_set_error("multi: %s -> %s", #call, (m)->nccl.error_string ? (m)->nccl.error_string(r__) : "NCCL error"); return TSP_ECUDA; } \
    } while (0)

extern "C" int tsp_multi_destroy(tsp_multi *m)
{
    if (!m) return TSP_OK;
    for (int i = 0; i < (int)m->h.size(); i++)
    {
        cudaSetDevice(m->dev[i]);
        cudaDeviceSynchronize();
        if (i < (int)m->d_b.size()) { cudaFree(m->d_b[i]); cudaFree(m->d_c[i]); }
        if (i < (int)m->stream.size() && m->stream[i]) cudaStreamDestroy(m->stream[i]);
        if (i < (int)m->comm.size() && m->comm[i]) m->nccl.comm_destroy(m->comm[i]);
        tsp_destroy(m->h[i]);
    }
    delete m;
    return TSP_OK;
}

extern "C" int tsp_multi_create(tsp_multi **out, int ndev, const int *devices, int precision)
{
    if (!out || ndev < 1 || ndev > 64 || !devices) { tsp_set_error("multi_create: bad argument"); return TSP_EINVAL; }
    *out = nullptr;
    for (int i = 0; i < ndev; i++)
        for (int j = 0; j < i; j++)
            if (devices[i] == devices[j]) { tsp_set_error("multi_create: device %d is listed twice", devices[i]); return TSP_EINVAL; }
    tsp_multi *m = new tsp_multi();
    m->ndev = ndev; m->precision = precision;
    m->dev.assign(devices, devices + ndev);
    int rc = TSP_OK;
    for (int i = 0; i < ndev && rc == TSP_OK; i++)
    {
        tsp_handle *h = nullptr;
        rc = tsp_create(&h, devices[i], precision);
        if (rc == TSP_OK) m->h.push_back(h);
    }
    m->d_b.assign(ndev, nullptr); m->d_c.assign(ndev, nullptr); m->b_bytes.assign(ndev, 0); m->c_bytes.assign(ndev, 0);
    m->stream.assign(ndev, nullptr); m->comm.assign(ndev, nullptr);
    for (int i = 0; i < ndev && rc == TSP_OK; i++)
    {
        if (cudaSetDevice(devices[i]) != cudaSuccess || cudaStreamCreateWithFlags(&m->stream[i], cudaStreamNonBlocking) != cudaSuccess)
        {
            tsp_set_error("multi_create: cannot create a stream on device %d", devices[i]);
            rc = TSP_ECUDA;
        }
    }
    if (rc == TSP_OK && ndev > 1)
    {
        rc = load_nccl(&m->nccl);
        if (rc == TSP_OK)
        {
            const int r = m->nccl.comm_init_all(m->comm.data(), ndev, devices);
            if (r != 0) { tsp_set_error("multi_create: ncclCommInitAll -> %s", m->nccl.error_string ? m->nccl.error_string(r) : "NCCL error"); rc = TSP_ECUDA; }
        }
    }
    if (rc != TSP_OK) { tsp_multi_destroy(m); return rc; }
    *out = m;
    return TSP_OK;
}

extern "C" int tsp_multi_device_count(const tsp_multi *m) { return m ? m->ndev : 0; }

extern "C" int tsp_multi_convert_host(tsp_multi *m, int rowA, int colA, long long nnz, const int *rp, const int *ci, const void *val,
                                      float gamma, float delta)
{
    if (!m || !rp) { tsp_set_error("multi_convert: null argument"); return TSP_EINVAL; }
    std::vector<int> rcs(m->ndev, TSP_OK);
    std::vector<std::string> errs(m->ndev);
    std::vector<std::thread> threads;
    for (int i = 0; i < m->ndev; i++)
        threads.emplace_back([&, i]() {
            rcs[i] = tsp_convert_host(m->h[i], rowA, colA, nnz, rp, ci, val, gamma, delta, i, m->ndev);
            if (rcs[i] != TSP_OK) errs[i] = tsp_last_error();   // the message is per thread: carry it over
        });
    for (auto &t : threads) t.join();
    for (int i = 0; i < m->ndev; i++)
        if (rcs[i] != TSP_OK) { tsp_set_error("multi_convert: device %d: %s", m->dev[i], errs[i].c_str()); return rcs[i]; }
    // the slabs must tile the rows in device order
    int at = 0;
    for (int i = 0; i < m->ndev; i++)
    {
        if (m->h[i]->row_begin != at && m->h[i]->row_begin != m->h[i]->row_end) { tsp_set_error("multi_convert: the row slabs of the devices do not tile the matrix"); return TSP_ESTATE; }
        if (m->h[i]->row_begin != m->h[i]->row_end) at = m->h[i]->row_end;
    }
    if (at != rowA) { tsp_set_error("multi_convert: the row slabs of the devices do not cover the matrix"); return TSP_ESTATE; }
    m->rowA = rowA; m->colA = colA; m->nnz = nnz; m->converted = true;
    return TSP_OK;
}

// info12: the per-class quantities of tsp_info summed over the devices; slabs2n[2*i], slabs2n[2*i+1]: first and
// one-past-last row of device i's slab of C (may be NULL).
extern "C" int tsp_multi_info(const tsp_multi *m, int *info12, int *slabs2n)
{
    if (!m || !info12) { tsp_set_error("multi_info: null argument"); return TSP_EINVAL; }
    memset(info12, 0, 12 * sizeof(int));
    for (int i = 0; i < m->ndev; i++)
    {
        int one[12], rows[2];
        TSP_TRY(tsp_info(m->h[i], one, rows));
        for (int k = 0; k < 12; k++) info12[k] += one[k];
        if (slabs2n) { slabs2n[2 * i] = rows[0]; slabs2n[2 * i + 1] = rows[1]; }
    }
    return TSP_OK;
}

static int ensure_buffers(tsp_multi *m, int colB)
{
    const size_t vsz = m->precision ? 4 : 2;
    const size_t per = ((size_t)m->colA + m->ndev - 1) / m->ndev;
    for (int i = 0; i < m->ndev; i++)
    {
        TSP_CUDA(cudaSetDevice(m->dev[i]));
        const size_t bb = per * m->ndev * colB * vsz, cb = (size_t)tsp_c_rows(m->h[i]) * colB * 4;
        if (bb > m->b_bytes[i]) { cudaFree(m->d_b[i]); m->d_b[i] = nullptr; m->b_bytes[i] = 0; TSP_CUDA(cudaMalloc(&m->d_b[i], bb)); m->b_bytes[i] = bb; }
        if (cb > m->c_bytes[i]) { cudaFree(m->d_c[i]); m->d_c[i] = nullptr; m->c_bytes[i] = 0; TSP_CUDA(cudaMalloc((void **)&m->d_c[i], cb)); m->c_bytes[i] = cb; }
    }
    return TSP_OK;
}

// every device uploads its own row block of B; the blocks are all-gathered in place into every device's copy
static int replicate_b(tsp_multi *m, const void *h_b, int colB)
{
    const size_t vsz = m->precision ? 4 : 2;
    const size_t per = ((size_t)m->colA + m->ndev - 1) / m->ndev, block = per * colB * vsz;
    for (int i = 0; i < m->ndev; i++)
    {
        const size_t lo = per * i < (size_t)m->colA ? per * i : (size_t)m->colA, hi = per * (i + 1) < (size_t)m->colA ? per * (i + 1) : (size_t)m->colA;
        TSP_CUDA(cudaSetDevice(m->dev[i]));
        if (hi > lo)
            TSP_CUDA(cudaMemcpyAsync((unsigned char *)m->d_b[i] + block * i, (const unsigned char *)h_b + lo * colB * vsz, (hi - lo) * colB * vsz,
                                     cudaMemcpyHostToDevice, m->stream[i]));
    }
    if (m->ndev > 1)
    {
        NCCL_TRY(m, m->nccl.group_start());
        for (int i = 0; i < m->ndev; i++)
            NCCL_TRY(m, m->nccl.all_gather((unsigned char *)m->d_b[i] + block * i, m->d_b[i], block, kNcclUint8, m->comm[i], m->stream[i]));
        NCCL_TRY(m, m->nccl.group_end());
    }
    return TSP_OK;
}

// One product with host operands: h_b is colA x colB_padded (value type), h_c receives rowA x colB_padded floats.
extern "C" int tsp_multi_spmm_host(tsp_multi *m, const void *h_b, float *h_c, int colB)
{
    if (!m || !h_b || !h_c) { tsp_set_error("multi_spmm_host: null argument"); return TSP_EINVAL; }
    if (!m->converted) { tsp_set_error("multi_spmm_host: convert first"); return TSP_ESTATE; }
    TSP_TRY(ensure_buffers(m, colB));
    TSP_TRY(replicate_b(m, h_b, colB));
    for (int i = 0; i < m->ndev; i++)
    {
        tsp_handle *h = m->h[i];
        TSP_TRY(tsp_spmm(h, m->d_b[i], m->d_c[i], colB, m->stream[i]));
        if (h->row_end > h->row_begin)
            TSP_CUDA(cudaMemcpyAsync(h_c + (size_t)h->row_begin * colB, m->d_c[i], (size_t)(h->row_end - h->row_begin) * colB * 4, cudaMemcpyDeviceToHost,
                                     m->stream[i]));
    }
    int rc = TSP_OK;
    for (int i = 0; i < m->ndev; i++)
    {
        const int r = tsp_check_error(m->h[i], m->stream[i]);
        if (r != TSP_OK && rc == TSP_OK) rc = r;
    }
    return rc;
}

// The upstream runtime driver (call_tilespmm_cuda, src/csr2tile.h:826-1093) over N devices: replicate B, tune every
// device's thresholds on its own shard, checked product into h_c (may be NULL), then `repeat` timed passes started on
// all devices together; time_ms is the slowest device's mean.  out6 = {best_th64, best_th16, best_th8 of device 0,
// pre_time_ms (cpu_pre_time_ms + tuning), time_ms, tflops = 2*nnz*colB_logical/time}.
extern "C" int tsp_multi_run(tsp_multi *m, const void *h_b, float *h_c, int colB, int colB_logical, double cpu_pre_ms, int repeat, double *out6)
{
    if (!m || !h_b || !out6 || repeat <= 0) { tsp_set_error("multi_run: bad argument"); return TSP_EINVAL; }
    if (!m->converted) { tsp_set_error("multi_run: convert first"); return TSP_ESTATE; }
    TSP_TRY(ensure_buffers(m, colB));
    TSP_TRY(replicate_b(m, h_b, colB));
    for (int i = 0; i < m->ndev; i++) { TSP_CUDA(cudaSetDevice(m->dev[i])); TSP_CUDA(cudaStreamSynchronize(m->stream[i])); }
    const double t_a = now_ms();
    std::vector<int> rcs(m->ndev, TSP_OK), best(3 * m->ndev, 32);
    std::vector<std::string> errs(m->ndev);
    {
        std::vector<std::thread> threads;
        for (int i = 0; i < m->ndev; i++)
            threads.emplace_back([&, i]() {
                float tune_ms = 0.f;
                rcs[i] = tsp_tune(m->h[i], m->d_b[i], m->d_c[i], colB, &best[3 * i], &tune_ms);
                if (rcs[i] != TSP_OK) errs[i] = tsp_last_error();
            });
        for (auto &t : threads) t.join();
    }
    for (int i = 0; i < m->ndev; i++)
        if (rcs[i] != TSP_OK) { tsp_set_error("multi_run: tuning on device %d: %s", m->dev[i], errs[i].c_str()); return rcs[i]; }
    const double tune_ms = now_ms() - t_a;
    if (h_c) TSP_TRY(tsp_multi_spmm_host(m, h_b, h_c, colB));
    // timed passes: every device runs `repeat` products on its stream, bracketed by its own events
    std::vector<cudaEvent_t> e0(m->ndev), e1(m->ndev);
    for (int i = 0; i < m->ndev; i++)
    {
        TSP_CUDA(cudaSetDevice(m->dev[i]));
        TSP_CUDA(cudaEventCreate(&e0[i])); TSP_CUDA(cudaEventCreate(&e1[i]));
        for (int w = 0; w < 20; w++) TSP_TRY(tsp_spmm(m->h[i], m->d_b[i], m->d_c[i], colB, m->stream[i]));
    }
    for (int i = 0; i < m->ndev; i++) { TSP_CUDA(cudaSetDevice(m->dev[i])); TSP_CUDA(cudaStreamSynchronize(m->stream[i])); }
    for (int i = 0; i < m->ndev; i++) { TSP_CUDA(cudaSetDevice(m->dev[i])); TSP_CUDA(cudaEventRecord(e0[i], m->stream[i])); }
    for (int p = 0; p < repeat; p++)
        for (int i = 0; i < m->ndev; i++) TSP_TRY(tsp_spmm(m->h[i], m->d_b[i], m->d_c[i], colB, m->stream[i]));
    double worst = 0.0;
    int rc = TSP_OK;
    for (int i = 0; i < m->ndev; i++)
    {
        TSP_CUDA(cudaSetDevice(m->dev[i]));
        TSP_CUDA(cudaEventRecord(e1[i], m->stream[i]));
        const int r = tsp_check_error(m->h[i], m->stream[i]);
        if (r != TSP_OK && rc == TSP_OK) rc = r;
        float ms = 0.f;
        TSP_CUDA(cudaEventElapsedTime(&ms, e0[i], e1[i]));
        if (ms / repeat > worst) worst = ms / repeat;
        cudaEventDestroy(e0[i]); cudaEventDestroy(e1[i]);
    }
    TSP_TRY(rc);
    out6[0] = best[0]; out6[1] = best[1]; out6[2] = best[2];
    out6[3] = cpu_pre_ms + tune_ms;
    out6[4] = worst;
    out6[5] = (2.0 * (double)m->nnz * 1.0e-6 / worst * colB_logical) / 1000.0;   // src/csr2tile.h:1057
    return TSP_OK;
}
