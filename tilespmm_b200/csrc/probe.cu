// Measurement aid: how fast this GPU can gather randomly chosen row segments of a dense matrix into its SMs.
//
// The SpMM kernels read every gathered row of B from L2 (B is read from HBM about once), so next to the HBM
// roofline they have a second ceiling: the rate at which all SMs together can pull scattered 128..512-byte
// segments out of L2.  This probe measures that rate with nothing else going on: each warp loads row segments
// named by a random index list with 16-byte loads, eight independent loads in flight per lane, and adds them up.
// No upstream counterpart.
#include "tsp_internal.cuh"

namespace
{

__global__ void k_probe_gather(const float4 *__restrict__ buf, const int *__restrict__ idx, long long nidx, int row_f4, float *out)
{
    // one warp-wide load covers 32 / row_f4 row segments of row_f4 * 16 bytes
    const int lane = threadIdx.x & 31, rpl = 32 / row_f4, sub = lane / row_f4, c = lane % row_f4;
    const long long warp = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5, nwarps = ((long long)gridDim.x * blockDim.x) >> 5;
    const long long per_iter = 8ll * rpl;
    float acc = 0.f;
    for (long long i = warp * per_iter; i + per_iter <= nidx; i += nwarps * per_iter)
    {
        // the indices of an iteration are one coalesced load, handed around by shuffles
        const int mine = lane < per_iter ? __ldg(idx + i + lane) : 0;
        float4 v[8];
#pragma unroll
        for (int j = 0; j < 8; j++) v[j] = __ldg(buf + (size_t)__shfl_sync(0xffffffffu, mine, j * rpl + sub) * row_f4 + c);
#pragma unroll
        for (int j = 0; j < 8; j++) acc += v[j].x + v[j].y + v[j].z + v[j].w;
    }
    if (acc == 123.456f) out[0] = acc;   // keeps the loads alive
}

}  // namespace

extern "C" int tsp_probe_gather(int device, int row_bytes, long long buffer_bytes, double *gb_per_s)
{
    if (!gb_per_s || (row_bytes != 128 && row_bytes != 256 && row_bytes != 512) || buffer_bytes < (1 << 20) || buffer_bytes > (8ll << 30))
    {
        tsp_set_error("probe_gather: row_bytes must be 128, 256 or 512 and the buffer between 1 MiB and 8 GiB");
        return TSP_EINVAL;
    }
    TSP_CUDA(cudaSetDevice(device));
    const int row_f4 = row_bytes / 16;
    const long long rows = buffer_bytes / row_bytes;
    const long long nidx = (1ll << 31) / row_bytes;   // 2 GiB gathered per launch
    float4 *buf = nullptr;
    int *idx = nullptr;
    float *out = nullptr;
    cudaEvent_t e0 = nullptr, e1 = nullptr;
    std::vector<int> h(nidx);
    unsigned long long s = 0x9e3779b97f4a7c15ull;   // xorshift: any fixed sequence will do
    for (auto &x : h) { s ^= s << 13; s ^= s >> 7; s ^= s << 17; x = (int)(s % (unsigned long long)rows); }
    int rc = TSP_OK;
    auto fail = [&](cudaError_t e) { if (e != cudaSuccess && rc == TSP_OK) { tsp_set_error("probe_gather: %s", cudaGetErrorString(e)); rc = e == cudaErrorMemoryAllocation ? TSP_ENOMEM : TSP_ECUDA; } };
    fail(cudaMalloc((void **)&buf, (size_t)rows * row_bytes));
    fail(cudaMalloc((void **)&idx, (size_t)nidx * 4));
    fail(cudaMalloc((void **)&out, 4));
    if (rc == TSP_OK)
    {
        fail(cudaMemset(buf, 0, (size_t)rows * row_bytes));
        fail(cudaMemcpy(idx, h.data(), (size_t)nidx * 4, cudaMemcpyHostToDevice));
        fail(cudaEventCreate(&e0));
        fail(cudaEventCreate(&e1));
    }
    if (rc == TSP_OK)
    {
        cudaDeviceProp prop;
        fail(cudaGetDeviceProperties(&prop, device));
        const int blocks = prop.multiProcessorCount * 8, reps = 10;
        for (int w = 0; w < 3; w++) k_probe_gather<<<blocks, 256>>>(buf, idx, nidx, row_f4, out);
        fail(cudaEventRecord(e0));
        for (int w = 0; w < reps; w++) k_probe_gather<<<blocks, 256>>>(buf, idx, nidx, row_f4, out);
        fail(cudaEventRecord(e1));
        fail(cudaEventSynchronize(e1));
        fail(cudaGetLastError());
        float ms = 0;
        if (rc == TSP_OK) fail(cudaEventElapsedTime(&ms, e0, e1));
        if (rc == TSP_OK) *gb_per_s = (double)nidx * row_bytes * reps / (ms * 1e6);
    }
    if (e0) cudaEventDestroy(e0);
    if (e1) cudaEventDestroy(e1);
    cudaFree(buf); cudaFree(idx); cudaFree(out);
    return rc;
}
