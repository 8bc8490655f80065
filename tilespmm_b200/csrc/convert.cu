// GPU partitioning and CSR -> tile conversion.
//
// Replaces upstream matrix_split (src/hetero_split.h:144-291) and Tile_create (src/csr2tile.h:724-795), which
// run on the host with per-thread column flag arrays.  Here every stage is a data-parallel kernel:
//
//   1. keys (8-row block, column) for every stored entry -> radix sort -> unique: the sorted distinct
//      columns of every 8-row block (U8 lists, contiguous, with offsets u8_ptr).
//   2. exact distinct-column counts of every 8/16/64-row window starting at a multiple of 8 rows
//      (|U8|, two-list and eight-list unions by binary search) -- the N8/N16/N64 of the upstream scan.
//   3. the upstream decision (64 / 16 / 8 rows) evaluated for EVERY 8-aligned start in parallel, with the
//      same float comparisons, then the greedy chain i <- i + step(i) resolved chunk-wise.
//   4. keys (panel, column) -> sort -> unique: sorted distinct columns of every panel; tiles per panel,
//      prefix sums (tile_ptr), tile_colidx with upstream's padding.
//   5. one warp per original row: rank of every entry in its panel's column list -> tile, slot; per-tile
//      entry counts (tile_nnz) and the dense tile values, accumulated in CSR order in value type.
//
// All outputs are bit-identical to upstream's for the same CSR, gamma and delta.
#include <cub/cub.cuh>

#include "tsp_internal.cuh"

namespace
{

constexpr int CHAIN_L = 512;  // 8-row blocks per chunk of the chain resolution

template <typename T>
struct DevBuf  // RAII device buffer for conversion scratch
{
    T *p = nullptr;
    size_t n = 0;
    int alloc(size_t count)
    {
        n = count;
        if (count == 0) count = 1;
        cudaError_t e = cudaMalloc((void **)&p, count * sizeof(T));
        if (e != cudaSuccess)
        {
            p = nullptr;
            tsp_set_error("conversion scratch: cudaMalloc of %zu bytes failed: %s", count * sizeof(T), cudaGetErrorString(e));
            return TSP_ENOMEM;
        }
        return TSP_OK;
    }
    void release() { if (p) cudaFree(p); p = nullptr; }
    ~DevBuf() { release(); }
};

__device__ __forceinline__ int lower_bound_dev(const int *a, int n, int key)
{
    int lo = 0, hi = n;
    while (lo < hi)
    {
        int mid = (lo + hi) >> 1;
        if (__ldg(a + mid) < key) lo = mid + 1; else hi = mid;
    }
    return lo;
}

// ---- stage 1

__global__ void k_make_block_keys(int rowA, const int *__restrict__ rowptr, const int *__restrict__ colidx,
                                  unsigned long long *__restrict__ keys)
{
    const int lane = threadIdx.x & 31;
    const int warps = (gridDim.x * blockDim.x) >> 5;
    for (int r = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; r < rowA; r += warps)
    {
        const int b = rowptr[r], e = rowptr[r + 1];
        const unsigned long long hi = (unsigned long long)(r >> 3) << 32;
        for (int j = b + lane; j < e; j += 32) keys[j] = hi | (unsigned int)colidx[j];
    }
}

// first index whose (key >> 32) >= g, for g = 0..ngroups
__global__ void k_group_offsets(const unsigned long long *__restrict__ keys, int n, int ngroups, int *__restrict__ ptr)
{
    int g = blockIdx.x * blockDim.x + threadIdx.x;
    if (g > ngroups) return;
    int lo = 0, hi = n;
    while (lo < hi)
    {
        int mid = (lo + hi) >> 1;
        if ((int)(keys[mid] >> 32) < g) lo = mid + 1; else hi = mid;
    }
    ptr[g] = lo;
}

__global__ void k_low_words(const unsigned long long *__restrict__ keys, int n, int *__restrict__ out)
{
    int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] = (int)(unsigned int)keys[i];
}

// ---- stage 2: distinct columns of windows of 2 and 8 consecutive blocks (one warp per window)

__global__ void k_window_counts(int nb8, int rowA, const int *__restrict__ u8_ptr, const int *__restrict__ ucols,
                                int *__restrict__ n16, int *__restrict__ n64, int want64)
{
    const int lane = threadIdx.x & 31;
    const int warps = (gridDim.x * blockDim.x) >> 5;
    for (int b = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; b < nb8; b += warps)
    {
        for (int pass = 0; pass < 2; pass++)
        {
            const int span = pass == 0 ? 2 : 8;
            if (pass == 1 && !want64) break;
            if ((long long)b * 8 + span * 8 > rowA) continue;  // upstream tests need the whole window inside the matrix
            const int g0 = u8_ptr[b], g1 = u8_ptr[b + span];
            int dup = 0;
            for (int g = g0 + lane; g < g1; g += 32)
            {
                int j = 1;
                while (j < span && g >= u8_ptr[b + j]) j++;
                j -= 1;  // the element belongs to block b + j
                const int col = ucols[g];
                for (int q = 0; q < j; q++)  // present in an earlier block of the window?
                {
                    const int s = u8_ptr[b + q], len = u8_ptr[b + q + 1] - s;
                    const int pos = lower_bound_dev(ucols + s, len, col);
                    if (pos < len && ucols[s + pos] == col) { dup++; break; }
                }
            }
            for (int o = 16; o > 0; o >>= 1) dup += __shfl_xor_sync(0xffffffffu, dup, o);
            if (lane == 0) (pass == 0 ? n16 : n64)[b] = (g1 - g0) - dup;
        }
    }
}

// ---- stage 3: the upstream decision at every 8-aligned start (src/hetero_split.h:196-276)

__global__ void k_decide(int nb8, int rowA, float gamma, float delta, int fixed, const int *__restrict__ u8_ptr,
                         const int *__restrict__ n16, const int *__restrict__ n64, unsigned char *__restrict__ cls_of)
{
    int b = blockIdx.x * blockDim.x + threadIdx.x;
    if (b >= nb8) return;
    if (fixed >= 0) { cls_of[b] = (unsigned char)fixed; return; }  // src/hetero_split.h:152-169
    const long long i = (long long)b * 8;
    int is64 = 0;
    if (gamma < 4.0f && i + 64 <= rowA)
    {
        const int N64 = n64[b];
        if (N64 > 0)
        {
            const float thr = gamma * N64;
            int s16 = 0;
            for (int q = 0; q < 4 && !is64; q++)
            {
                s16 += n16[b + 2 * q];
                if ((float)s16 > thr) is64 = 1;
            }
        }
    }
    if (is64) { cls_of[b] = 0; return; }
    int is16 = 0;
    if (delta <= 0.0f) is16 = 1;
    else if (!(delta > 2.0f) && i + 16 <= rowA)
    {
        const int N16 = n16[b];
        if (N16 > 0)
        {
            const float thr = delta * N16;
            int s8 = u8_ptr[b + 1] - u8_ptr[b];
            if ((float)s8 >= thr) is16 = 1;
            else
            {
                s8 += u8_ptr[b + 2] - u8_ptr[b + 1];
                if ((float)s8 >= thr) is16 = 1;
            }
        }
    }
    cls_of[b] = is16 ? 1 : 2;
}

__device__ __forceinline__ int step_of(int cls) { return cls == 0 ? 8 : (cls == 1 ? 2 : 1); }

// For every chunk of CHAIN_L blocks and every entry offset 0..7: where the chain leaves the chunk and how
// many panels of each class it creates inside.
__global__ void k_chain_local(int nb8, int nchunk, const unsigned char *__restrict__ cls_of, unsigned char *__restrict__ exit_off,
                              int *__restrict__ counts /* [nchunk*8][3] */)
{
    int t = blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= nchunk * 8) return;
    const int c = t >> 3, o = t & 7;
    long long pos = (long long)c * CHAIN_L + o;
    const long long end = min((long long)(c + 1) * CHAIN_L, (long long)nb8);
    int cnt[3] = {0, 0, 0};
    while (pos < end)
    {
        const int k = cls_of[pos];
        cnt[k]++;
        pos += step_of(k);
    }
    long long off = pos - (long long)(c + 1) * CHAIN_L;
    exit_off[t] = (unsigned char)(off < 0 ? 0 : (off > 7 ? 7 : off));
    counts[t * 3 + 0] = cnt[0]; counts[t * 3 + 1] = cnt[1]; counts[t * 3 + 2] = cnt[2];
}

// Sequential composition over chunks (one thread; nchunk is rows/4096).
__global__ void k_chain_compose(int nchunk, const unsigned char *__restrict__ exit_off, const int *__restrict__ counts,
                                int *__restrict__ entry, int *__restrict__ base /* [nchunk+1][3] */)
{
    if (blockIdx.x || threadIdx.x) return;
    int e = 0, run[3] = {0, 0, 0};
    for (int c = 0; c < nchunk; c++)
    {
        entry[c] = e;
        base[c * 3 + 0] = run[0]; base[c * 3 + 1] = run[1]; base[c * 3 + 2] = run[2];
        const int t = c * 8 + e;
        run[0] += counts[t * 3 + 0]; run[1] += counts[t * 3 + 1]; run[2] += counts[t * 3 + 2];
        e = exit_off[t];
    }
    base[nchunk * 3 + 0] = run[0]; base[nchunk * 3 + 1] = run[1]; base[nchunk * 3 + 2] = run[2];
}

// Walk every chunk from its true entry and emit the panels in scan order.
__global__ void k_chain_emit(int nb8, int nchunk, int rowA, const unsigned char *__restrict__ cls_of, const int *__restrict__ entry,
                             const int *__restrict__ base, const int *__restrict__ rowptr, int *__restrict__ seq_blk,
                             unsigned char *__restrict__ seq_cls, int *__restrict__ seq_idx, int *__restrict__ blk_seq,
                             unsigned long long *__restrict__ class_rows_nnz /* [3][2] */)
{
    int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= nchunk) return;
    long long pos = (long long)c * CHAIN_L + entry[c];
    const long long end = min((long long)(c + 1) * CHAIN_L, (long long)nb8);
    int idx[3] = {base[c * 3 + 0], base[c * 3 + 1], base[c * 3 + 2]};
    int seq = idx[0] + idx[1] + idx[2];
    unsigned long long rows[3] = {0, 0, 0}, nnz[3] = {0, 0, 0};
    while (pos < end)
    {
        const int k = cls_of[pos], st = step_of(k);
        seq_blk[seq] = (int)pos;
        seq_cls[seq] = (unsigned char)k;
        seq_idx[seq] = idx[k]++;
        for (int q = 0; q < st && pos + q < nb8; q++) blk_seq[pos + q] = seq;
        const long long r0 = pos * 8, r1 = min(r0 + st * 8, (long long)rowA);
        rows[k] += (unsigned long long)(r1 - r0);
        nnz[k] += (unsigned long long)(rowptr[r1] - rowptr[r0]);
        seq++;
        pos += st;
    }
    for (int k = 0; k < 3; k++)
        if (rows[k])
        {
            atomicAdd(&class_rows_nnz[k * 2 + 0], rows[k]);
            atomicAdd(&class_rows_nnz[k * 2 + 1], nnz[k]);
        }
}

// ---- stage 4

__global__ void k_make_panel_keys(const unsigned long long *__restrict__ ukeys, int n, const int *__restrict__ blk_seq,
                                  unsigned long long *__restrict__ out)
{
    int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const unsigned long long k = ukeys[i];
    out[i] = ((unsigned long long)blk_seq[(int)(k >> 32)] << 32) | (k & 0xffffffffull);
}

__global__ void k_seq_tiles(int nseq, const int *__restrict__ pptr, const unsigned char *__restrict__ seq_cls, int precision,
                            int *__restrict__ seq_tiles)
{
    int s = blockIdx.x * blockDim.x + threadIdx.x;
    if (s >= nseq) return;
    const int bn = tsp_bn(precision, seq_cls[s]);
    seq_tiles[s] = (pptr[s + 1] - pptr[s] + bn - 1) / bn;  // src/csr2tile.h:45-46
}

// scatter the per-panel tile counts and first rows of the shard [s0, s1) into the per-class arrays
__global__ void k_class_arrays(int s0, int s1, const int *__restrict__ seq_tiles, const unsigned char *__restrict__ seq_cls,
                               const int *__restrict__ seq_idx, const int *__restrict__ seq_blk, int p0_64, int p0_16, int p0_8,
                               int *cnt64, int *cnt16, int *cnt8, int *row64, int *row16, int *row8)
{
    int s = s0 + blockIdx.x * blockDim.x + threadIdx.x;
    if (s >= s1) return;
    const int k = seq_cls[s];
    const int p = seq_idx[s] - (k == 0 ? p0_64 : (k == 1 ? p0_16 : p0_8));
    (k == 0 ? cnt64 : (k == 1 ? cnt16 : cnt8))[p] = seq_tiles[s];
    (k == 0 ? row64 : (k == 1 ? row16 : row8))[p] = seq_blk[s] * 8;
}

// tile_colidx: sorted distinct columns, the tail padded with the panel's last column (src/csr2tile.h:117-132)
__global__ void k_fill_colidx(int s0, int s1, int precision, const int *__restrict__ pptr, const int *__restrict__ pcols,
                              const unsigned char *__restrict__ seq_cls, const int *__restrict__ seq_idx, int p0_64, int p0_16, int p0_8,
                              const int *__restrict__ tp64, const int *__restrict__ tp16, const int *__restrict__ tp8,
                              int *__restrict__ ci64, int *__restrict__ ci16, int *__restrict__ ci8)
{
    const int lane = threadIdx.x & 31;
    const int warps = (gridDim.x * blockDim.x) >> 5;
    for (int s = s0 + ((blockIdx.x * blockDim.x + threadIdx.x) >> 5); s < s1; s += warps)
    {
        const int k = seq_cls[s], bn = tsp_bn(precision, k);
        const int p = seq_idx[s] - (k == 0 ? p0_64 : (k == 1 ? p0_16 : p0_8));
        const int *tp = k == 0 ? tp64 : (k == 1 ? tp16 : tp8);
        int *ci = k == 0 ? ci64 : (k == 1 ? ci16 : ci8);
        const int t0 = tp[p], nt = tp[p + 1] - t0;
        if (nt == 0) continue;
        const int g0 = pptr[s], d = pptr[s + 1] - g0;
        const int last = pcols[g0 + d - 1];
        int *dst = ci + (size_t)t0 * bn;
        for (int q = lane; q < nt * bn; q += 32) dst[q] = q < d ? pcols[g0 + q] : last;
    }
}

// ---- stage 5: values and per-tile entry counts, one warp per original row

template <typename V>
__device__ __forceinline__ V add_in_value_type(V a, V b);
template <>
__device__ __forceinline__ __half add_in_value_type<__half>(__half a, __half b) { return __hadd(a, b); }
template <>
__device__ __forceinline__ float add_in_value_type<float>(float a, float b) { return __fadd_rn(a, b); }

template <typename V>
__global__ void k_place_values(int rowA, int precision, int s0, int s1, const int *__restrict__ rowptr, const int *__restrict__ colidx,
                               const V *__restrict__ val, const int *__restrict__ blk_seq, const unsigned char *__restrict__ seq_cls,
                               const int *__restrict__ seq_idx, const int *__restrict__ seq_blk, const int *__restrict__ pptr,
                               const int *__restrict__ pcols, int p0_64, int p0_16, int p0_8, const int *__restrict__ tp64,
                               const int *__restrict__ tp16, const int *__restrict__ tp8, int *tn64, int *tn16, int *tn8,
                               V *v64, V *v16, V *v8)
{
    const int lane = threadIdx.x & 31;
    const int warps = (gridDim.x * blockDim.x) >> 5;
    for (int r = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; r < rowA; r += warps)
    {
        const int s = blk_seq[r >> 3];
        if (s < s0 || s >= s1) continue;
        const int jb = rowptr[r], je = rowptr[r + 1];
        if (jb == je) continue;
        const int k = seq_cls[s], bm = tsp_bm(k), bn = tsp_bn(precision, k);
        const int p = seq_idx[s] - (k == 0 ? p0_64 : (k == 1 ? p0_16 : p0_8));
        const int t0 = (k == 0 ? tp64 : (k == 1 ? tp16 : tp8))[p];
        int *tn = k == 0 ? tn64 : (k == 1 ? tn16 : tn8);
        V *vals = k == 0 ? v64 : (k == 1 ? v16 : v8);
        const int ri = r - seq_blk[s] * 8;
        const int g0 = pptr[s], d = pptr[s + 1] - g0;
        for (int base = jb; base < je; base += 32)
        {
            const int j = base + lane;
            const bool active = j < je;
            unsigned long long pos = ~0ull - (unsigned long long)lane;  // never equal between lanes
            V v = V(0.0f);
            if (active)
            {
                const int rank = lower_bound_dev(pcols + g0, d, colidx[j]);
                const int t = rank / bn, c = rank - t * bn;
                atomicAdd(&tn[t0 + t], 1);
                pos = (unsigned long long)(t0 + t) * (unsigned long long)(bm * bn) + (unsigned long long)tsp_device_index(precision, k, ri, c);
                v = val[j];
            }
            // Repeated (row, col) entries land on one position and must be added in CSR order
            // (src/csr2tile.h:271, 283, 318): the lowest lane of every group of equal positions adds the
            // group's values in lane order.
            const unsigned int grp = __match_any_sync(0xffffffffu, pos);
            const bool leader = active && (__ffs(grp) - 1) == lane;
            int most = __popc(grp);
            for (int o = 16; o > 0; o >>= 1) most = max(most, __shfl_xor_sync(0xffffffffu, most, o));
            V acc = V(0.0f);
            if (leader) acc = vals[pos];
            unsigned int rest = grp;
            for (int q = 0; q < most; q++)
            {
                const int src = rest ? __ffs(rest) - 1 : lane;
                const V got = __shfl_sync(0xffffffffu, v, src);
                if (leader && rest) acc = add_in_value_type<V>(acc, got);
                rest &= rest - 1;
            }
            if (leader) vals[pos] = acc;
            __syncwarp();
        }
    }
}

// 64-row tiles back to the upstream order (sub-blocks in mma.sync fragment order, src/csr2tile.h:319-372)
template <typename V>
__global__ void k_export64(int precision, long long nelem, const V *__restrict__ src, V *__restrict__ dst)
{
    const int bn = tsp_bn(precision, 0), per = 64 * bn;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < nelem; i += (long long)gridDim.x * blockDim.x)
    {
        const long long tile = i / per;
        const int e = (int)(i - tile * per), r = e / bn, c = e - r * bn;
        dst[tile * per + tsp_upstream_index(precision, 0, r, c)] = src[tile * per + tsp_umma_index(precision, r, c)];
    }
}

inline int blocks_for(long long n, int threads) { return (int)((n + threads - 1) / threads > 0 ? (n + threads - 1) / threads : 1); }

int sort_unique_keys(DevBuf<unsigned long long> &keys, DevBuf<unsigned long long> &tmp, int n, int key_bits, int *n_unique)
{
    // radix sort on the bits in use, then unique; result left in `keys`
    DevBuf<unsigned char> scratch;
    DevBuf<int> d_count;
    TSP_TRY(d_count.alloc(1));
    size_t bytes_sort = 0, bytes_uniq = 0;
    cub::DoubleBuffer<unsigned long long> db(keys.p, tmp.p);
    TSP_CUDA(cub::DeviceRadixSort::SortKeys(nullptr, bytes_sort, db, n, 0, key_bits));
    TSP_CUDA(cub::DeviceSelect::Unique(nullptr, bytes_uniq, keys.p, tmp.p, d_count.p, n));
    TSP_TRY(scratch.alloc(bytes_sort > bytes_uniq ? bytes_sort : bytes_uniq));
    TSP_CUDA(cub::DeviceRadixSort::SortKeys(scratch.p, bytes_sort, db, n, 0, key_bits));
    unsigned long long *sorted = db.Current(), *other = db.Alternate();
    TSP_CUDA(cub::DeviceSelect::Unique(scratch.p, bytes_uniq, sorted, other, d_count.p, n));
    TSP_CUDA(cudaMemcpy(n_unique, d_count.p, sizeof(int), cudaMemcpyDeviceToHost));
    if (other != keys.p) { unsigned long long *t = keys.p; keys.p = tmp.p; tmp.p = t; }
    return TSP_OK;
}

int bits_for(unsigned long long v)
{
    int b = 1;
    while (b < 64 && (v >> b)) b++;
    return b;
}

}  // namespace

void tsp_free_tiles(tsp_handle *h)
{
    for (int k = 0; k < 3; k++)
    {
        TspClass &c = h->cls[k];
        cudaFree(c.d_tile_ptr); cudaFree(c.d_tile_nnz); cudaFree(c.d_tile_colidx); cudaFree(c.d_panel_row); cudaFree(c.d_val);
        cudaFree(c.d_task_row); cudaFree(c.d_task_start); cudaFree(c.d_split_row); cudaFree(c.d_task_count); cudaFree(c.d_task_pack);
        c = TspClass();
        c.BM = tsp_bm(k);
        c.BN = tsp_bn(h->precision, k);
    }
    h->converted = false;
    h->bmap_ptr = nullptr;
}

int tsp_export_values_upstream(const tsp_handle *h, int cls, void *h_dst)
{
    const TspClass &c = h->cls[cls];
    const size_t vsz = h->precision ? 4 : 2;
    const long long nelem = (long long)c.tilenum * c.BM * c.BN;
    if (nelem == 0) return TSP_OK;
    if (cls != 0)
    {
        TSP_CUDA(cudaMemcpy(h_dst, c.d_val, nelem * vsz, cudaMemcpyDeviceToHost));
        return TSP_OK;
    }
    DevBuf<unsigned char> tmp;
    TSP_TRY(tmp.alloc(nelem * vsz));
    const int blocks = (int)(nelem / 256 + 1 > 65535 ? 65535 : nelem / 256 + 1);
    if (h->precision == 0) k_export64<__half><<<blocks, 256>>>(0, nelem, (const __half *)c.d_val, (__half *)tmp.p);
    else k_export64<float><<<blocks, 256>>>(1, nelem, (const float *)c.d_val, (float *)tmp.p);
    TSP_CUDA(cudaGetLastError());
    TSP_CUDA(cudaMemcpy(h_dst, tmp.p, nelem * vsz, cudaMemcpyDeviceToHost));
    return TSP_OK;
}

int tsp_convert_impl(tsp_handle *h, int rowA, int colA, long long nnz64, const int *d_rowptr, const int *d_colidx,
                     const void *d_val, float gamma, float delta, int shard_index, int shard_count)
{
    if (rowA <= 0 || colA <= 0 || nnz64 < 0 || nnz64 > 0x7fffffffLL || shard_count < 1 || shard_index < 0 || shard_index >= shard_count)
    {
        tsp_set_error("convert: bad shape or shard (rowA=%d colA=%d nnz=%lld shard %d/%d)", rowA, colA, nnz64, shard_index, shard_count);
        return TSP_EINVAL;
    }
    TSP_CUDA(cudaSetDevice(h->device));
    tsp_free_tiles(h);
    h->rowA = rowA; h->colA = colA; h->nnzA = nnz64;
    const int nnz = (int)nnz64;
    const int prec = h->precision;
    const int nb8 = (rowA + 7) / 8;
    const int T = 256;

    int fixed = -1;  // src/hetero_split.h:152-169
    if (gamma <= 0.0f) fixed = 0;
    else if (gamma >= 4.0f && delta <= 0.0f) fixed = 1;
    else if (gamma >= 4.0f && delta > 2.0f) fixed = 2;
    const bool want64 = fixed < 0 && gamma < 4.0f;
    const bool want16 = fixed < 0 && (want64 || (delta > 0.0f && !(delta > 2.0f)));

    // ---- stage 1: sorted distinct columns of every 8-row block
    DevBuf<unsigned long long> keys, keys_tmp;
    DevBuf<int> u8_ptr, ucols;
    TSP_TRY(keys.alloc(nnz)); TSP_TRY(keys_tmp.alloc(nnz)); TSP_TRY(u8_ptr.alloc((size_t)nb8 + 9));
    int nu = 0;
    if (nnz > 0)
    {
        k_make_block_keys<<<blocks_for((long long)rowA * 32, T) > 65535 * 4 ? 65535 * 4 : blocks_for((long long)rowA * 32, T), T>>>(rowA, d_rowptr, d_colidx, keys.p);
        TSP_CUDA(cudaGetLastError());
        TSP_TRY(sort_unique_keys(keys, keys_tmp, nnz, 32 + bits_for((unsigned long long)nb8), &nu));
    }
    k_group_offsets<<<blocks_for(nb8 + 1, T), T>>>(keys.p, nu, nb8, u8_ptr.p);
    TSP_CUDA(cudaGetLastError());
    // windows near the end index u8_ptr past nb8: pad with the total
    {
        std::vector<int> pad(8, nu);
        TSP_CUDA(cudaMemcpy(u8_ptr.p + nb8 + 1, pad.data(), 8 * sizeof(int), cudaMemcpyHostToDevice));
    }
    TSP_TRY(ucols.alloc(nu));
    if (nu) k_low_words<<<blocks_for(nu, T), T>>>(keys.p, nu, ucols.p);
    TSP_CUDA(cudaGetLastError());

    // ---- stage 2 + 3: window counts, decisions, chain
    DevBuf<int> n16, n64, entry, base, counts, seq_blk, seq_idx, blk_seq;
    DevBuf<unsigned char> cls_of, exit_off, seq_cls;
    DevBuf<unsigned long long> class_rows_nnz;
    TSP_TRY(n16.alloc(nb8)); TSP_TRY(n64.alloc(nb8)); TSP_TRY(cls_of.alloc(nb8));
    if (want16 || want64)
    {
        TSP_CUDA(cudaMemset(n16.p, 0, (size_t)nb8 * 4)); TSP_CUDA(cudaMemset(n64.p, 0, (size_t)nb8 * 4));
        const int blocks = blocks_for((long long)nb8 * 32, T) > 148 * 64 ? 148 * 64 : blocks_for((long long)nb8 * 32, T);
        k_window_counts<<<blocks, T>>>(nb8, rowA, u8_ptr.p, ucols.p, n16.p, n64.p, want64 ? 1 : 0);
        TSP_CUDA(cudaGetLastError());
    }
    k_decide<<<blocks_for(nb8, T), T>>>(nb8, rowA, gamma, delta, fixed, u8_ptr.p, n16.p, n64.p, cls_of.p);
    TSP_CUDA(cudaGetLastError());
    const int nchunk = (nb8 + CHAIN_L - 1) / CHAIN_L;
    TSP_TRY(exit_off.alloc((size_t)nchunk * 8)); TSP_TRY(counts.alloc((size_t)nchunk * 24)); TSP_TRY(entry.alloc(nchunk));
    TSP_TRY(base.alloc((size_t)nchunk * 3 + 3));
    k_chain_local<<<blocks_for((long long)nchunk * 8, T), T>>>(nb8, nchunk, cls_of.p, exit_off.p, counts.p);
    k_chain_compose<<<1, 32>>>(nchunk, exit_off.p, counts.p, entry.p, base.p);
    TSP_CUDA(cudaGetLastError());
    int totals[3];
    TSP_CUDA(cudaMemcpy(totals, base.p + (size_t)nchunk * 3, sizeof(totals), cudaMemcpyDeviceToHost));
    const int nseq = totals[0] + totals[1] + totals[2];
    TSP_TRY(seq_blk.alloc(nseq)); TSP_TRY(seq_cls.alloc(nseq)); TSP_TRY(seq_idx.alloc(nseq)); TSP_TRY(blk_seq.alloc(nb8));
    TSP_TRY(class_rows_nnz.alloc(6));
    TSP_CUDA(cudaMemset(class_rows_nnz.p, 0, 6 * sizeof(unsigned long long)));
    k_chain_emit<<<blocks_for(nchunk, 128), 128>>>(nb8, nchunk, rowA, cls_of.p, entry.p, base.p, d_rowptr, seq_blk.p, seq_cls.p,
                                                  seq_idx.p, blk_seq.p, class_rows_nnz.p);
    TSP_CUDA(cudaGetLastError());

    // ---- stage 4: sorted distinct columns of every panel
    DevBuf<int> pptr_buf, pcols_buf, seq_tiles;
    const int *pptr = nullptr, *pcols = nullptr;
    const bool all8 = totals[0] == 0 && totals[1] == 0;
    if (all8) { pptr = u8_ptr.p; pcols = ucols.p; }  // an 8-row panel is one 8-row block
    else
    {
        int np = 0;
        if (nu)
        {
            k_make_panel_keys<<<blocks_for(nu, T), T>>>(keys.p, nu, blk_seq.p, keys_tmp.p);
            TSP_CUDA(cudaGetLastError());
            { unsigned long long *t = keys.p; keys.p = keys_tmp.p; keys_tmp.p = t; }
            TSP_TRY(sort_unique_keys(keys, keys_tmp, nu, 32 + bits_for((unsigned long long)nseq), &np));
        }
        TSP_TRY(pptr_buf.alloc((size_t)nseq + 1)); TSP_TRY(pcols_buf.alloc(np));
        k_group_offsets<<<blocks_for(nseq + 1, T), T>>>(keys.p, np, nseq, pptr_buf.p);
        if (np) k_low_words<<<blocks_for(np, T), T>>>(keys.p, np, pcols_buf.p);
        TSP_CUDA(cudaGetLastError());
        pptr = pptr_buf.p; pcols = pcols_buf.p;
        ucols.release();
    }
    keys.release(); keys_tmp.release();
    TSP_TRY(seq_tiles.alloc(nseq));
    if (nseq) k_seq_tiles<<<blocks_for(nseq, T), T>>>(nseq, pptr, seq_cls.p, prec, seq_tiles.p);
    TSP_CUDA(cudaGetLastError());

    // ---- shard selection: a contiguous range of the panel sequence, balanced by tile bytes
    std::vector<int> h_seq_tiles(nseq), h_seq_blk(nseq), h_seq_idx(nseq);
    std::vector<unsigned char> h_seq_cls(nseq);
    if (nseq)
    {
        TSP_CUDA(cudaMemcpy(h_seq_tiles.data(), seq_tiles.p, (size_t)nseq * 4, cudaMemcpyDeviceToHost));
        TSP_CUDA(cudaMemcpy(h_seq_blk.data(), seq_blk.p, (size_t)nseq * 4, cudaMemcpyDeviceToHost));
        TSP_CUDA(cudaMemcpy(h_seq_idx.data(), seq_idx.p, (size_t)nseq * 4, cudaMemcpyDeviceToHost));
        TSP_CUDA(cudaMemcpy(h_seq_cls.data(), seq_cls.p, (size_t)nseq, cudaMemcpyDeviceToHost));
    }
    int s0 = 0, s1 = nseq;
    if (shard_count > 1)
    {
        const size_t vsz = prec ? 4 : 2;
        std::vector<double> prefix((size_t)nseq + 1, 0.0);
        for (int s = 0; s < nseq; s++)
        {
            const int k = h_seq_cls[s], bm = tsp_bm(k), bn = tsp_bn(prec, k);
            // bytes of one tile (values + indices + gathered rows of a 128-wide B) plus the C rows of the panel and a
            // fixed 12 KB per panel: measured on R-MAT scale 24, starting a task costs about as much as 3 more tiles
            prefix[s + 1] = prefix[s] + (double)h_seq_tiles[s] * (bm * bn * vsz + bn * 4 + bn * 128 * vsz) + bm * 128 * 4.0 + 12288.0;
        }
        auto cut = [&](int g) {
            const double want = prefix[nseq] * g / shard_count;
            int lo = 0, hi = nseq;
            while (lo < hi) { int mid = (lo + hi) / 2; if (prefix[mid] < want) lo = mid + 1; else hi = mid; }
            return lo;
        };
        s0 = shard_index == 0 ? 0 : cut(shard_index);
        s1 = shard_index == shard_count - 1 ? nseq : cut(shard_index + 1);
        if (s1 < s0) s1 = s0;
    }
    h->row_begin = s0 < nseq ? h_seq_blk[s0] * 8 : rowA;
    h->row_end = s1 < nseq ? h_seq_blk[s1] * 8 : rowA;
    if (s0 == s1) h->row_begin = h->row_end;

    int p0[3] = {0, 0, 0}, p1[3] = {0, 0, 0};
    {
        bool seen[3] = {false, false, false};
        for (int k = 0; k < 3; k++) { p0[k] = -1; p1[k] = -1; }
        for (int s = s0; s < s1; s++)
        {
            const int k = h_seq_cls[s];
            if (!seen[k]) { seen[k] = true; p0[k] = h_seq_idx[s]; }
            p1[k] = h_seq_idx[s] + 1;
        }
        for (int k = 0; k < 3; k++) if (!seen[k]) { p0[k] = 0; p1[k] = 0; }
    }
    for (int k = 0; k < 3; k++)
    {
        TspClass &c = h->cls[k];
        c.tilem = p1[k] - p0[k];
        TSP_CUDA(cudaMalloc((void **)&c.d_tile_ptr, ((size_t)c.tilem + 1) * 4));
        TSP_CUDA(cudaMemset(c.d_tile_ptr, 0, ((size_t)c.tilem + 1) * 4));
        TSP_CUDA(cudaMalloc((void **)&c.d_panel_row, ((size_t)c.tilem + 1) * 4));
    }
    if (s1 > s0)
    {
        k_class_arrays<<<blocks_for(s1 - s0, T), T>>>(s0, s1, seq_tiles.p, seq_cls.p, seq_idx.p, seq_blk.p, p0[0], p0[1], p0[2],
                                                      h->cls[0].d_tile_ptr, h->cls[1].d_tile_ptr, h->cls[2].d_tile_ptr,
                                                      h->cls[0].d_panel_row, h->cls[1].d_panel_row, h->cls[2].d_panel_row);
        TSP_CUDA(cudaGetLastError());
    }
    for (int k = 0; k < 3; k++)
    {
        TspClass &c = h->cls[k];
        size_t bytes = 0;
        TSP_CUDA(cub::DeviceScan::ExclusiveSum(nullptr, bytes, c.d_tile_ptr, c.d_tile_ptr, c.tilem + 1));
        DevBuf<unsigned char> scratch;
        TSP_TRY(scratch.alloc(bytes));
        TSP_CUDA(cub::DeviceScan::ExclusiveSum(scratch.p, bytes, c.d_tile_ptr, c.d_tile_ptr, c.tilem + 1));
        c.h_tile_ptr.resize((size_t)c.tilem + 1);
        c.h_panel_row.resize(c.tilem);
        TSP_CUDA(cudaMemcpy(c.h_tile_ptr.data(), c.d_tile_ptr, ((size_t)c.tilem + 1) * 4, cudaMemcpyDeviceToHost));
        if (c.tilem) TSP_CUDA(cudaMemcpy(c.h_panel_row.data(), c.d_panel_row, (size_t)c.tilem * 4, cudaMemcpyDeviceToHost));
        c.tilenum = c.h_tile_ptr[c.tilem];
        // rows and nnz of the class inside the shard
        c.rows = 0; c.nnz = 0;
        const size_t vsz = prec ? 4 : 2;
        TSP_CUDA(cudaMalloc((void **)&c.d_tile_nnz, ((size_t)c.tilenum + 1) * 4));
        TSP_CUDA(cudaMemset(c.d_tile_nnz, 0, ((size_t)c.tilenum + 1) * 4));
        TSP_CUDA(cudaMalloc((void **)&c.d_tile_colidx, ((size_t)c.tilenum * c.BN + 1) * 4));
        TSP_CUDA(cudaMalloc((void **)&c.d_val, (size_t)c.tilenum * c.BM * c.BN * vsz + 16));
        TSP_CUDA(cudaMemset(c.d_val, 0, (size_t)c.tilenum * c.BM * c.BN * vsz + 16));
    }
    // class rows / nnz: whole-matrix totals come from the chain; per-shard ones from the host panel lists
    {
        std::vector<int> h_rowptr_ends;  // only needed per shard: compute on device totals when unsharded
        unsigned long long tot[6];
        TSP_CUDA(cudaMemcpy(tot, class_rows_nnz.p, sizeof(tot), cudaMemcpyDeviceToHost));
        if (shard_count == 1)
            for (int k = 0; k < 3; k++) { h->cls[k].rows = (int)tot[k * 2]; h->cls[k].nnz = (long long)tot[k * 2 + 1]; }
        else
        {
            std::vector<int> h_rowptr((size_t)rowA + 1);
            TSP_CUDA(cudaMemcpy(h_rowptr.data(), d_rowptr, ((size_t)rowA + 1) * 4, cudaMemcpyDeviceToHost));
            for (int k = 0; k < 3; k++)
                for (int p = 0; p < h->cls[k].tilem; p++)
                {
                    const int r0 = h->cls[k].h_panel_row[p], r1 = r0 + h->cls[k].BM < rowA ? r0 + h->cls[k].BM : rowA;
                    h->cls[k].rows += r1 - r0;
                    h->cls[k].nnz += h_rowptr[r1] - h_rowptr[r0];
                }
        }
    }
    if (s1 > s0)
    {
        const int blocks = blocks_for((long long)(s1 - s0) * 32, T) > 148 * 32 ? 148 * 32 : blocks_for((long long)(s1 - s0) * 32, T);
        k_fill_colidx<<<blocks, T>>>(s0, s1, prec, pptr, pcols, seq_cls.p, seq_idx.p, p0[0], p0[1], p0[2], h->cls[0].d_tile_ptr,
                                     h->cls[1].d_tile_ptr, h->cls[2].d_tile_ptr, h->cls[0].d_tile_colidx, h->cls[1].d_tile_colidx,
                                     h->cls[2].d_tile_colidx);
        TSP_CUDA(cudaGetLastError());
        // ---- stage 5
        const int vblocks = blocks_for((long long)rowA * 32, T) > 148 * 64 ? 148 * 64 : blocks_for((long long)rowA * 32, T);
        if (prec == 0)
            k_place_values<__half><<<vblocks, T>>>(rowA, 0, s0, s1, d_rowptr, d_colidx, (const __half *)d_val, blk_seq.p, seq_cls.p, seq_idx.p,
                                                   seq_blk.p, pptr, pcols, p0[0], p0[1], p0[2], h->cls[0].d_tile_ptr, h->cls[1].d_tile_ptr,
                                                   h->cls[2].d_tile_ptr, h->cls[0].d_tile_nnz, h->cls[1].d_tile_nnz, h->cls[2].d_tile_nnz,
                                                   (__half *)h->cls[0].d_val, (__half *)h->cls[1].d_val, (__half *)h->cls[2].d_val);
        else
            k_place_values<float><<<vblocks, T>>>(rowA, 1, s0, s1, d_rowptr, d_colidx, (const float *)d_val, blk_seq.p, seq_cls.p, seq_idx.p,
                                                  seq_blk.p, pptr, pcols, p0[0], p0[1], p0[2], h->cls[0].d_tile_ptr, h->cls[1].d_tile_ptr,
                                                  h->cls[2].d_tile_ptr, h->cls[0].d_tile_nnz, h->cls[1].d_tile_nnz, h->cls[2].d_tile_nnz,
                                                  (float *)h->cls[0].d_val, (float *)h->cls[1].d_val, (float *)h->cls[2].d_val);
        TSP_CUDA(cudaGetLastError());
    }
    for (int k = 0; k < 3; k++)  // tile_nnz: exclusive scan over tilenum+1 entries (src/csr2tile.h:786)
    {
        TspClass &c = h->cls[k];
        size_t bytes = 0;
        TSP_CUDA(cub::DeviceScan::ExclusiveSum(nullptr, bytes, c.d_tile_nnz, c.d_tile_nnz, c.tilenum + 1));
        DevBuf<unsigned char> scratch;
        TSP_TRY(scratch.alloc(bytes));
        TSP_CUDA(cub::DeviceScan::ExclusiveSum(scratch.p, bytes, c.d_tile_nnz, c.d_tile_nnz, c.tilenum + 1));
    }
    TSP_CUDA(cudaDeviceSynchronize());
    h->converted = true;
    return TSP_OK;
}
