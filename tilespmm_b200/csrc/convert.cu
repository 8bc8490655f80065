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
//      entry counts (tile_nnz); for the 16- and 8-row classes the dense tile values, accumulated in CSR order in
//      value type; for the 64-row class the row masks of every tile (bitmap).
//   6. 64-row class: entries per tile from the masks -> record sizes (packed: masks + values, dense: 4 KB) ->
//      prefix sum (record offsets) -> values placed in mask order (repeated entries summed in CSR order).
//
// tile_ptr, tile_nnz, tile_colidx, panel rows and, after expansion (tsp_export), the tile values are bit-identical to
// upstream's for the same CSR, gamma and delta; the masks are defined by the CSR alone (an explicit zero sets its bit).
//
// Host side: all scratch comes from a workspace kept in the handle (no cudaMalloc/cudaFree per stage), the tile
// arrays of all classes are one allocation, and the host reads back a handful of scalars in three small copies.
#include <cub/cub.cuh>
#include <stdlib.h>
#include <sys/time.h>

#include "tsp_internal.cuh"

namespace
{

constexpr int CHAIN_L = 64;   // 8-row blocks per chunk of the chain resolution

// Bump allocator over the handle's workspace chunks.  The first conversion sizes chunk 0 from nnz and rowA; what
// does not fit (sizes known only later) goes into further chunks, which later conversions reuse.
struct Workspace
{
    tsp_handle *h;
    size_t chunk = 0, used = 0;
    explicit Workspace(tsp_handle *hh) : h(hh) {}
    template <typename T>
    int get(T **p, size_t count)
    {
        size_t bytes = (count * sizeof(T) + 255) & ~(size_t)255;
        if (bytes == 0) bytes = 256;
        while (chunk < h->ws_chunks.size() && h->ws_chunks[chunk].second - used < bytes) { chunk++; used = 0; }
        if (chunk == h->ws_chunks.size())
        {
            void *q = nullptr;
            const size_t cap = bytes > ((size_t)8 << 20) ? bytes : ((size_t)8 << 20);
            cudaError_t e = cudaMalloc(&q, cap);
            if (e != cudaSuccess)
            {
                tsp_set_error("conversion workspace: cudaMalloc of %zu bytes failed: %s", cap, cudaGetErrorString(e));
                return TSP_ENOMEM;
            }
            h->ws_chunks.push_back({q, cap});
            used = 0;
        }
        *p = reinterpret_cast<T *>(static_cast<unsigned char *>(h->ws_chunks[chunk].first) + used);
        used += bytes;
        return TSP_OK;
    }
};

int reserve_workspace(tsp_handle *h, size_t bytes)
{
    if (!h->ws_chunks.empty() && h->ws_chunks[0].second >= bytes) return TSP_OK;
    tsp_free_workspace(h);
    void *q = nullptr;
    cudaError_t e = cudaMalloc(&q, bytes);
    if (e != cudaSuccess)
    {
        tsp_set_error("conversion workspace: cudaMalloc of %zu bytes failed: %s", bytes, cudaGetErrorString(e));
        return TSP_ENOMEM;
    }
    h->ws_chunks.push_back({q, bytes});
    return TSP_OK;
}

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

// Keys of all entries, and the consistency check of the CSR: row pointers start at 0, never decrease and end at nnz,
// every column lies in [0, colA).  A CSR that fails is reported through *bad before anything is indexed with its
// contents (the row ranges used here are clamped to [0, nnz]); every slot of keys[] is written for a valid CSR.
__global__ void k_make_block_keys(int rowA, int colA, int nnz, const int *__restrict__ rowptr, const int *__restrict__ colidx,
                                  unsigned long long *__restrict__ keys, int *__restrict__ bad)
{
    const int lane = threadIdx.x & 31;
    const int warps = (gridDim.x * blockDim.x) >> 5;
    int wrong = 0;
    for (int r = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; r < rowA; r += warps)
    {
        int b = rowptr[r], e = rowptr[r + 1];
        if (b > e || b < 0 || e > nnz || (r == 0 && b != 0) || (r == rowA - 1 && e != nnz)) wrong = 1;
        b = min(max(b, 0), nnz); e = min(max(e, b), nnz);
        const unsigned long long hi = (unsigned long long)(r >> 3) << 32;
        for (int j = b + lane; j < e; j += 32)
        {
            const int c = colidx[j];
            if (c < 0 || c >= colA) wrong = 1;
            keys[j] = hi | (unsigned int)c;
        }
    }
    if (wrong) atomicExch(bad, 1);
}

// first index whose (key >> 32) >= g, for g = 0..ngroups (+ `pad` more entries holding the total)
__global__ void k_group_offsets(const unsigned long long *__restrict__ keys, const int *__restrict__ n_ptr, int ngroups, int pad,
                                int *__restrict__ ptr)
{
    int g = blockIdx.x * blockDim.x + threadIdx.x;
    if (g > ngroups + pad) return;
    const int n = *n_ptr;
    if (g > ngroups) { ptr[g] = n; return; }
    int lo = 0, hi = n;
    while (lo < hi)
    {
        int mid = (lo + hi) >> 1;
        if ((int)(keys[mid] >> 32) < g) lo = mid + 1; else hi = mid;
    }
    ptr[g] = lo;
}

__global__ void k_low_words(const unsigned long long *__restrict__ keys, const int *__restrict__ n_ptr, int *__restrict__ out)
{
    const int n = *n_ptr;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) out[i] = (int)(unsigned int)keys[i];
}

// ---- stage 2: distinct columns of windows of 2 and 8 consecutive blocks
//
// A column that occurs in block j counts once in every window [b, b+span) that contains j but not the previous block p
// that holds the same column: b in (max(p, j-span), j].  So every (block, column) pair adds +1 at max(p, j-span)+1 and -1
// at j+1 of a difference array, and a prefix sum gives the exact distinct count of every window.  The previous block of
// every pair comes from one more radix sort, by (column, block).  Work is linear in the number of pairs, whatever the
// row lengths (a warp per window with searches in the earlier lists took 39 ms on a scale-20 R-MAT graph; this takes 2).

__global__ void k_col_block_keys(const unsigned long long *__restrict__ ukeys, int n, int block_bits, unsigned long long *__restrict__ out)
{
    int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const unsigned long long k = ukeys[i];
    out[i] = ((k & 0xffffffffull) << block_bits) | (k >> 32);
}

__global__ void k_window_diffs(const unsigned long long *__restrict__ by_col, int n, int block_bits, int want64, int *__restrict__ d16,
                               int *__restrict__ d64)
{
    int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const unsigned long long mask = (1ull << block_bits) - 1ull, k = by_col[i];
    const int j = (int)(k & mask);
    int p = -1;
    if (i > 0)
    {
        const unsigned long long q = by_col[i - 1];
        if ((q >> block_bits) == (k >> block_bits)) p = (int)(q & mask);
    }
    atomicAdd(&d16[max(p, j - 2) + 1], 1);
    atomicAdd(&d16[j + 1], -1);
    if (want64)
    {
        atomicAdd(&d64[max(p, j - 8) + 1], 1);
        atomicAdd(&d64[j + 1], -1);
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

// The greedy chain i <- i + step(i) is resolved chunk-wise.  Chunks are short (CHAIN_L blocks) and staged in shared
// memory, so that a walk costs shared-memory latency per step; the chunks are then linked by a parallel scan over
// "entry offset -> exit offset" tables (8 states), not by a serial pass.

// For every chunk of CHAIN_L blocks and every entry offset 0..7: where the chain leaves the chunk and how
// many panels of each class it creates inside.  One thread per (chunk, entry); 32 chunks per block of 256 threads.
__global__ void __launch_bounds__(256)
k_chain_local(int nb8, int nchunk, const unsigned char *__restrict__ cls_of, unsigned char *__restrict__ exit_off,
              int *__restrict__ counts /* [nchunk*8][3] */)
{
    __shared__ unsigned char cls_s[32 * CHAIN_L];
    const long long first = (long long)blockIdx.x * 32 * CHAIN_L;
    for (int i = threadIdx.x; i < 32 * CHAIN_L; i += 256) cls_s[i] = first + i < nb8 ? cls_of[first + i] : 2;
    __syncthreads();
    const int t = blockIdx.x * 256 + threadIdx.x;
    if (t >= nchunk * 8) return;
    const int c = t >> 3, o = t & 7, lc = threadIdx.x >> 3;
    const int len = (int)min((long long)CHAIN_L, (long long)nb8 - (long long)c * CHAIN_L);
    int pos = o, cnt[3] = {0, 0, 0};
    while (pos < len)
    {
        const int k = cls_s[lc * CHAIN_L + pos];
        cnt[k]++;
        pos += step_of(k);
    }
    const int off = pos - CHAIN_L;
    exit_off[t] = (unsigned char)(off < 0 ? 0 : (off > 7 ? 7 : off));
    counts[t * 3 + 0] = cnt[0]; counts[t * 3 + 1] = cnt[1]; counts[t * 3 + 2] = cnt[2];
}

// Links the chunks: the entry offset of every chunk (composition of the chunks' transition tables, 8 states of 3 bits
// packed into one word) and the number of panels of each class before it.  One block; scans by composition.
__global__ void __launch_bounds__(1024)
k_chain_compose(int nchunk, const unsigned char *__restrict__ exit_off, const int *__restrict__ counts, int *__restrict__ entry,
                int *__restrict__ base /* [nchunk+1][3] */)
{
    __shared__ unsigned int warp_f[32];
    __shared__ int warp_n[32][3];
    __shared__ unsigned int carry_state;
    __shared__ int carry_n[3];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    // f(state) for all 8 states in one word; compose(f, g)(x) = g(f(x)) -- f first
    auto apply = [](unsigned int f, unsigned int x) { return (f >> (3 * x)) & 7u; };
    auto compose = [&](unsigned int f, unsigned int g) {
        unsigned int h = 0;
#pragma unroll
        for (unsigned int x = 0; x < 8; x++) h |= apply(g, apply(f, x)) << (3 * x);
        return h;
    };
    constexpr unsigned int IDENT = 0u | 1u << 3 | 2u << 6 | 3u << 9 | 4u << 12 | 5u << 15 | 6u << 18 | 7u << 21;
    if (threadIdx.x == 0) { carry_state = 0; carry_n[0] = carry_n[1] = carry_n[2] = 0; }
    __syncthreads();
    for (int base_c = 0; base_c < nchunk; base_c += 1024)
    {
        const int c = base_c + threadIdx.x;
        unsigned int f = IDENT;
        if (c < nchunk)
        {
            f = 0;
            for (unsigned int x = 0; x < 8; x++) f |= (unsigned int)exit_off[c * 8 + x] << (3 * x);
        }
        // inclusive scan of the transition tables over the 1024 chunks of this pass
        unsigned int incl = f;
        for (int o = 1; o < 32; o <<= 1) { const unsigned int y = __shfl_up_sync(0xffffffffu, incl, o); if (lane >= o) incl = compose(y, incl); }
        if (lane == 31) warp_f[warp] = incl;
        __syncthreads();
        if (warp == 0)
        {
            unsigned int w = warp_f[lane];
            for (int o = 1; o < 32; o <<= 1) { const unsigned int y = __shfl_up_sync(0xffffffffu, w, o); if (lane >= o) w = compose(y, w); }
            warp_f[lane] = w;
        }
        __syncthreads();
        // exclusive prefix function of this chunk: everything before it in this pass
        unsigned int excl = __shfl_up_sync(0xffffffffu, incl, 1);
        if (lane == 0) excl = IDENT;
        if (warp > 0) excl = compose(warp_f[warp - 1], excl);
        const unsigned int e = apply(excl, carry_state);       // the true entry offset of chunk c
        int n[3] = {0, 0, 0};
        if (c < nchunk)
        {
            entry[c] = (int)e;
            const int t = c * 8 + (int)e;
            n[0] = counts[t * 3 + 0]; n[1] = counts[t * 3 + 1]; n[2] = counts[t * 3 + 2];
        }
        // exclusive prefix sums of the panel counts along the true path
        int in[3] = {n[0], n[1], n[2]};
        for (int o = 1; o < 32; o <<= 1)
#pragma unroll
            for (int k = 0; k < 3; k++) { const int y = __shfl_up_sync(0xffffffffu, in[k], o); if (lane >= o) in[k] += y; }
        if (lane == 31) { warp_n[warp][0] = in[0]; warp_n[warp][1] = in[1]; warp_n[warp][2] = in[2]; }
        __syncthreads();
        if (warp == 0)
        {
            int w[3] = {warp_n[lane][0], warp_n[lane][1], warp_n[lane][2]};
            for (int o = 1; o < 32; o <<= 1)
#pragma unroll
                for (int k = 0; k < 3; k++) { const int y = __shfl_up_sync(0xffffffffu, w[k], o); if (lane >= o) w[k] += y; }
            warp_n[lane][0] = w[0]; warp_n[lane][1] = w[1]; warp_n[lane][2] = w[2];
        }
        __syncthreads();
        if (c < nchunk)
#pragma unroll
            for (int k = 0; k < 3; k++) base[c * 3 + k] = carry_n[k] + (warp ? warp_n[warp - 1][k] : 0) + in[k] - n[k];
        __syncthreads();
        if (threadIdx.x == 1023)   // totals of this pass -> carry for the next
        {
            carry_state = apply(compose(excl, f), carry_state);
#pragma unroll
            for (int k = 0; k < 3; k++) carry_n[k] += warp_n[31][k];
        }
        __syncthreads();
    }
    if (threadIdx.x == 0) { base[nchunk * 3 + 0] = carry_n[0]; base[nchunk * 3 + 1] = carry_n[1]; base[nchunk * 3 + 2] = carry_n[2]; }
}

// Walk every chunk from its true entry and emit the panels in scan order.  One thread per chunk, 128 chunks per block.
__global__ void __launch_bounds__(128)
k_chain_emit(int nb8, int nchunk, int rowA, const unsigned char *__restrict__ cls_of, const int *__restrict__ entry,
             const int *__restrict__ base, const int *__restrict__ rowptr, int *__restrict__ seq_blk,
             unsigned char *__restrict__ seq_cls, int *__restrict__ seq_idx, int *__restrict__ blk_seq,
             unsigned long long *__restrict__ class_rows_nnz /* [3][2] */)
{
    __shared__ unsigned char cls_s[128 * CHAIN_L];
    const long long first = (long long)blockIdx.x * 128 * CHAIN_L;
    for (int i = threadIdx.x; i < 128 * CHAIN_L; i += 128) cls_s[i] = first + i < nb8 ? cls_of[first + i] : 2;
    __syncthreads();
    int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= nchunk) return;
    long long pos = (long long)c * CHAIN_L + entry[c];
    const long long end = min((long long)(c + 1) * CHAIN_L, (long long)nb8);
    int idx[3] = {base[c * 3 + 0], base[c * 3 + 1], base[c * 3 + 2]};
    int seq = idx[0] + idx[1] + idx[2];
    unsigned long long rows[3] = {0, 0, 0}, nnz[3] = {0, 0, 0};
    while (pos < end)
    {
        const int k = cls_s[pos - first], st = step_of(k);
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

// ---- shard selection on the device: a contiguous range of the panel sequence, balanced by tile bytes

// bytes of one tile (values + indices + gathered rows of a 128-wide B) plus the C rows of the panel and a fixed
// 12 KB per panel: measured on R-MAT scale 24, starting a task costs about as much as 3 more tiles
__global__ void k_panel_costs(int nseq, int precision, const int *__restrict__ seq_tiles, const unsigned char *__restrict__ seq_cls,
                              double *__restrict__ cost)
{
    int s = blockIdx.x * blockDim.x + threadIdx.x;
    if (s >= nseq) return;
    const int k = seq_cls[s], bm = tsp_bm(k), bn = tsp_bn(precision, k), vsz = precision ? 4 : 2;
    cost[s] = (double)seq_tiles[s] * (bm * bn * vsz + bn * 4 + bn * 128 * vsz) + bm * 128 * 4.0 + 12288.0;
}

// out[0..1] = s0, s1 (panel range of the shard), out[2..4] / out[5..7] = first / one-past-last class-local panel index
// (initialised here, completed by k_shard_bounds), out[8..9] = first / one-past-last original row of the shard
__global__ void k_find_cuts(int nseq, int rowA, int shard_index, int shard_count, const double *__restrict__ prefix /* inclusive */,
                            const int *__restrict__ seq_blk, int *__restrict__ out)
{
    if (blockIdx.x || threadIdx.x) return;
    const double total = nseq ? prefix[nseq - 1] : 0.0;
    auto cut = [&](int g) {   // first s whose exclusive prefix is >= total * g / shard_count
        const double want = total * g / shard_count;
        int lo = 0, hi = nseq;
        while (lo < hi) { const int mid = (lo + hi) / 2; const double ex = mid ? prefix[mid - 1] : 0.0; if (ex < want) lo = mid + 1; else hi = mid; }
        return lo;
    };
    int s0 = shard_index == 0 ? 0 : cut(shard_index);
    int s1 = shard_index == shard_count - 1 ? nseq : cut(shard_index + 1);
    if (s1 < s0) s1 = s0;
    out[0] = s0; out[1] = s1;
    for (int k = 0; k < 3; k++) { out[2 + k] = 0x7fffffff; out[5 + k] = 0; }
    int rb = s0 < nseq ? seq_blk[s0] * 8 : rowA, re = s1 < nseq ? seq_blk[s1] * 8 : rowA;
    if (s0 == s1) rb = re;
    out[8] = rb; out[9] = re;
}

__global__ void k_shard_bounds(const int *cuts, const unsigned char *__restrict__ seq_cls, const int *__restrict__ seq_idx, int *out)
{
    const int s0 = cuts[0], s1 = cuts[1];
    for (int s = s0 + blockIdx.x * blockDim.x + threadIdx.x; s < s1; s += gridDim.x * blockDim.x)
    {
        const int k = seq_cls[s];
        atomicMin(&out[2 + k], seq_idx[s]);
        atomicMax(&out[5 + k], seq_idx[s] + 1);
    }
}

// rows and stored entries of every class inside the shard
__global__ void k_class_totals(int s0, int s1, int rowA, const unsigned char *__restrict__ seq_cls, const int *__restrict__ seq_blk,
                               const int *__restrict__ rowptr, unsigned long long *__restrict__ rows_nnz /* [3][2] */)
{
    unsigned long long rows[3] = {0, 0, 0}, nnz[3] = {0, 0, 0};
    for (int s = s0 + blockIdx.x * blockDim.x + threadIdx.x; s < s1; s += gridDim.x * blockDim.x)
    {
        const int k = seq_cls[s];
        const long long r0 = (long long)seq_blk[s] * 8, r1 = min(r0 + tsp_bm(k), (long long)rowA);
        rows[k] += (unsigned long long)(r1 - r0);
        nnz[k] += (unsigned long long)(rowptr[r1] - rowptr[r0]);
    }
    for (int k = 0; k < 3; k++)
        if (rows[k]) { atomicAdd(&rows_nnz[k * 2], rows[k]); atomicAdd(&rows_nnz[k * 2 + 1], nnz[k]); }
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

// Repeated (row, col) entries land on one position and must be added in CSR order (src/csr2tile.h:271, 283, 318):
// the lowest lane of every group of equal positions adds the group's values in lane order, starting from what the
// position already holds.  Called by all lanes of a warp; inactive lanes pass a position no other lane has.
template <typename V>
__device__ __forceinline__ void add_in_csr_order(V *vals, unsigned long long pos, V v, bool active, int lane)
{
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

// One warp per original row: tile and slot of every entry; per-tile entry counts (all classes); dense tile values of
// the 16- and 8-row classes; row masks of the 64-row tiles.
template <typename V>
__global__ void k_place_values(int rowA, int precision, int s0, int s1, const int *__restrict__ rowptr, const int *__restrict__ colidx,
                               const V *__restrict__ val, const int *__restrict__ blk_seq, const unsigned char *__restrict__ seq_cls,
                               const int *__restrict__ seq_idx, const int *__restrict__ seq_blk, const int *__restrict__ pptr,
                               const int *__restrict__ pcols, int p0_64, int p0_16, int p0_8, const int *__restrict__ tp64,
                               const int *__restrict__ tp16, const int *__restrict__ tp8, int *tn64, int *tn16, int *tn8,
                               unsigned int *__restrict__ mask64 /* 32-bit words of the row masks */, V *v16, V *v8)
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
        V *vals = k == 1 ? v16 : v8;
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
                if (k == 0)
                {
                    // row mask of (tile, row): 16-bit masks (TF32) are addressed as halves of 32-bit words
                    const size_t bit = ((size_t)(t0 + t) * 64 + ri) * bn + c;
                    atomicOr(&mask64[bit >> 5], 1u << (bit & 31));
                }
                else
                {
                    pos = (unsigned long long)(t0 + t) * (unsigned long long)(bm * bn) + (unsigned long long)tsp_upstream_index(precision, k, ri, c);
                    v = val[j];
                }
            }
            if (k != 0) add_in_csr_order<V>(vals, pos, v, active, lane);
        }
    }
}

// ---- stage 6: packed records of the 64-row class

// One warp per tile: entries of the tile from its masks -> record size in 16-byte units (dense 4 KB record above
// TSP_REC_MAX_VALS values), the dense flag, and the number of values before every row (row_off, 64 per tile).
__global__ void k_rec_sizes(int tilenum, int precision, const unsigned int *__restrict__ mask64, unsigned int *__restrict__ units,
                            unsigned char *__restrict__ dense, unsigned short *__restrict__ row_off)
{
    const int lane = threadIdx.x & 31;
    const int warps = (gridDim.x * blockDim.x) >> 5;
    const int vsz = precision ? 4 : 2, max_vals = TSP_REC_MAX_VALS(precision);
    for (int t = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; t < tilenum; t += warps)
    {
        // lane l owns rows 2l and 2l+1
        unsigned int w0, w1;
        if (precision) { const unsigned int w = mask64[(size_t)t * 32 + lane]; w0 = w & 0xffffu; w1 = w >> 16; }
        else { w0 = mask64[(size_t)t * 64 + 2 * lane]; w1 = mask64[(size_t)t * 64 + 2 * lane + 1]; }
        const int c0 = __popc(w0), cnt = c0 + __popc(w1);
        int incl = cnt;
        for (int o = 1; o < 32; o <<= 1) { const int y = __shfl_up_sync(0xffffffffu, incl, o); if (lane >= o) incl += y; }
        const int total = __shfl_sync(0xffffffffu, incl, 31);
        row_off[(size_t)t * 64 + 2 * lane] = (unsigned short)(incl - cnt);
        row_off[(size_t)t * 64 + 2 * lane + 1] = (unsigned short)(incl - cnt + c0);
        if (lane == 0)
        {
            const bool is_dense = total > max_vals;
            dense[t] = is_dense ? 1 : 0;
            units[t] = is_dense ? (64u * tsp_bn(precision, 0) * vsz) / 16u : tsp_packed_units(precision, total);
        }
    }
}

// rec[t] = exclusive prefix of the record sizes with the dense flag in bit 31; rec[tilenum] = total; units[] holds the
// exclusive prefix on entry.
__global__ void k_rec_finish(int tilenum, const unsigned int *__restrict__ prefix, const unsigned char *__restrict__ dense,
                             unsigned int *__restrict__ rec)
{
    int t = blockIdx.x * blockDim.x + threadIdx.x;
    if (t > tilenum) return;
    rec[t] = prefix[t] | (t < tilenum && dense[t] ? 0x80000000u : 0u);
}

// The position slots of every packed record start as 0xffff ("no entry"); the padding keeps that value.
__global__ void k_init_positions(int tilenum, int precision, const unsigned int *__restrict__ rec, unsigned char *__restrict__ pack)
{
    const int per = 2 + (precision ? 4 : 2);
    for (int t = blockIdx.x; t < tilenum; t += gridDim.x)
    {
        const unsigned int r = rec[t];
        if (r >> 31) continue;
        const unsigned int n_pad = ((rec[t + 1] & 0x7fffffffu) - r) * 16u / per;
        unsigned short *posn = reinterpret_cast<unsigned short *>(pack + (size_t)r * 16);
        for (unsigned int i = threadIdx.x; i < n_pad; i += blockDim.x) posn[i] = 0xffffu;
    }
}

// One warp per original row of the 64-row class: every entry's value goes to its place in the tile's record -- for a
// packed record the slot given by the masks (row-major order of the set bits), together with the entry's position in
// the operand tile; for a dense record the operand position itself.
template <typename V>
__global__ void k_place_values64(int rowA, int precision, int s0, int s1, const int *__restrict__ rowptr, const int *__restrict__ colidx,
                                 const V *__restrict__ val, const int *__restrict__ blk_seq, const unsigned char *__restrict__ seq_cls,
                                 const int *__restrict__ seq_idx, const int *__restrict__ seq_blk, const int *__restrict__ pptr,
                                 const int *__restrict__ pcols, int p0_64, const int *__restrict__ tp64, const unsigned int *__restrict__ mask64,
                                 const unsigned short *__restrict__ row_off, const unsigned int *__restrict__ rec, V *pack)
{
    const int lane = threadIdx.x & 31;
    const int warps = (gridDim.x * blockDim.x) >> 5;
    const int bn = tsp_bn(precision, 0), per16 = 16 / (int)sizeof(V), per = 2 + (int)sizeof(V);
    for (int r = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; r < rowA; r += warps)
    {
        const int s = blk_seq[r >> 3];
        if (s < s0 || s >= s1 || seq_cls[s] != 0) continue;
        const int jb = rowptr[r], je = rowptr[r + 1];
        if (jb == je) continue;
        const int t0 = tp64[seq_idx[s] - p0_64];
        const int ri = r - seq_blk[s] * 8;
        const int g0 = pptr[s], d = pptr[s + 1] - g0;
        for (int base = jb; base < je; base += 32)
        {
            const int j = base + lane;
            const bool active = j < je;
            unsigned long long pos = ~0ull - (unsigned long long)lane;
            V v = V(0.0f);
            if (active)
            {
                const int rank = lower_bound_dev(pcols + g0, d, colidx[j]);
                const int t = t0 + rank / bn, c = rank % bn;
                const unsigned int rw = rec[t];
                const unsigned long long rec_elem = (unsigned long long)(rw & 0x7fffffffu) * per16;
                if (rw >> 31) pos = rec_elem + (unsigned long long)tsp_umma_index(precision, ri, c);
                else
                {
                    const size_t bit = ((size_t)t * 64 + ri) * bn;          // first bit of the row mask
                    unsigned int m = mask64[bit >> 5] >> (bit & 31);
                    if (precision) m &= 0xffffu;
                    const unsigned int n_pad = ((rec[t + 1] & 0x7fffffffu) - rw) * 16u / per;
                    const unsigned int slot = row_off[(size_t)t * 64 + ri] + __popc(m & ((1u << c) - 1u));
                    // positions first (2 bytes each), then the values: n_pad * 2 bytes is a multiple of 16
                    pos = rec_elem + (unsigned long long)(n_pad * 2u / sizeof(V)) + slot;
                    reinterpret_cast<unsigned short *>(pack + (size_t)rw * per16)[slot] = (unsigned short)tsp_umma_index(precision, ri, c);
                }
                v = val[j];
            }
            add_in_csr_order<V>(pack, pos, v, active, lane);
        }
    }
}

// 64-row tiles as upstream stores them (dense, sub-blocks in mma.sync fragment order, src/csr2tile.h:319-372), expanded
// from the records; dst is zero-filled by the caller.  One warp per tile, lane l owns rows 2l and 2l+1.
template <typename V>
__global__ void k_export64(int tilenum, int precision, const unsigned int *__restrict__ rec, const unsigned char *__restrict__ pack,
                           V *__restrict__ dst)
{
    const int lane = threadIdx.x & 31;
    const int warps = (gridDim.x * blockDim.x) >> 5;
    const int bn = tsp_bn(precision, 0), per = 64 * bn;
    for (int t = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; t < tilenum; t += warps)
    {
        const unsigned int rw = rec[t];
        const unsigned char *record = pack + (size_t)(rw & 0x7fffffffu) * 16;
        V *out = dst + (size_t)t * per;
        if (rw >> 31)
        {
            const V *src = reinterpret_cast<const V *>(record);
            for (int e = lane; e < per; e += 32) { const int r = e / bn, c = e - r * bn; out[tsp_upstream_index(precision, 0, r, c)] = src[tsp_umma_index(precision, r, c)]; }
            continue;
        }
        // packed: positions (operand order) and values; the inverse of tsp_umma_index gives (row, column)
        const int per_rec = 2 + (int)sizeof(V), T = 16 / (int)sizeof(V);
        const unsigned int n_pad = ((rec[t + 1] & 0x7fffffffu) - rw) * 16u / per_rec;
        const unsigned short *posn = reinterpret_cast<const unsigned short *>(record);
        const V *src = reinterpret_cast<const V *>(record + n_pad * 2);
        for (unsigned int i = lane; i < n_pad; i += 32)
        {
            const unsigned int u = posn[i];
            if (u == 0xffffu) continue;
            const int core = u / (8 * T), r = ((core & 7) << 3) + (u % (8 * T)) / T, c = (core >> 3) * T + u % T;
            out[tsp_upstream_index(precision, 0, r, c)] = src[i];
        }
    }
}

inline int blocks_for(long long n, int threads) { return (int)((n + threads - 1) / threads > 0 ? (n + threads - 1) / threads : 1); }

// Radix sort on the bits in use, then unique.  keys/tmp are swapped so that the result is in `keys`; the number of
// distinct keys is left in *d_count (device).
int sort_unique_keys(unsigned long long *&keys, unsigned long long *&tmp, int n, int key_bits, void *scratch, size_t scratch_bytes,
                     int *d_count)
{
    cub::DoubleBuffer<unsigned long long> db(keys, tmp);
    size_t bytes = scratch_bytes;
    TSP_CUDA(cub::DeviceRadixSort::SortKeys(scratch, bytes, db, n, 0, key_bits));
    unsigned long long *sorted = db.Current(), *other = db.Alternate();
    bytes = scratch_bytes;
    TSP_CUDA(cub::DeviceSelect::Unique(scratch, bytes, sorted, other, d_count, n));
    keys = other; tmp = sorted;
    return TSP_OK;
}

size_t sort_unique_scratch_bytes(int n)
{
    size_t a = 0, b = 0;
    cub::DoubleBuffer<unsigned long long> db(nullptr, nullptr);
    cub::DeviceRadixSort::SortKeys(nullptr, a, db, n, 0, 64);
    cub::DeviceSelect::Unique(nullptr, b, (unsigned long long *)nullptr, (unsigned long long *)nullptr, (int *)nullptr, n);
    size_t c = 0, d = 0;   // the prefix sums over panels share the same scratch
    cub::DeviceScan::ExclusiveSum(nullptr, c, (int *)nullptr, (int *)nullptr, n + 1);
    cub::DeviceScan::InclusiveSum(nullptr, d, (double *)nullptr, (double *)nullptr, n + 1);
    if (b > a) a = b;
    if (c > a) a = c;
    if (d > a) a = d;
    return a + 256;
}

int bits_for(unsigned long long v)
{
    int b = 1;
    while (b < 64 && (v >> b)) b++;
    return b;
}

// small pinned host buffer for scalar read-backs
int pinned(tsp_handle *h, int **p)
{
    if (!h->h_pin) TSP_CUDA(cudaMallocHost(&h->h_pin, 4096));
    *p = static_cast<int *>(h->h_pin);
    return TSP_OK;
}

}  // namespace

void tsp_free_workspace(tsp_handle *h)
{
    for (auto &c : h->ws_chunks) cudaFree(c.first);
    h->ws_chunks.clear();
}

void tsp_free_tiles(tsp_handle *h, bool release)
{
    if (release)
    {
        cudaFree(h->tile_block); cudaFree(h->pack_block);
        h->tile_block = h->pack_block = nullptr;
        h->tile_block_bytes = h->pack_block_bytes = 0;
    }
    for (int k = 0; k < 3; k++)
    {
        TspClass &c = h->cls[k];
        TspClass fresh;
        if (release) { cudaFree(c.d_task_row); cudaFree(c.d_task_start); cudaFree(c.d_split_row); cudaFree(c.d_task_count); cudaFree(c.d_task_pack); }
        else
        {
            // the schedule arrays and their capacities survive: cudaFree/cudaMalloc per conversion cost more than the conversion kernels
            fresh.d_task_row = c.d_task_row; fresh.d_task_start = c.d_task_start; fresh.d_split_row = c.d_split_row;
            fresh.d_task_count = c.d_task_count; fresh.d_task_pack = c.d_task_pack;
            fresh.cap_tasks = c.cap_tasks; fresh.cap_panels = c.cap_panels;
        }
        c = fresh;
        c.BM = tsp_bm(k);
        c.BN = tsp_bn(h->precision, k);
    }
    h->converted = false;
    h->bmap_ptr = nullptr;
}

// One allocation for every tile array of the three classes; sizes come from cls[k].tilem and cls[k].tilenum.
// tile_ptr (inputs of a scan), tile_nnz (atomic counters), the dense values and the masks start as zeros.
int tsp_alloc_tile_arrays(tsp_handle *h)
{
    const size_t vsz = h->precision ? 4 : 2;
    size_t off = 0;
    auto take = [&](size_t bytes) { const size_t at = off; off += (bytes + 255) & ~(size_t)255; return at; };
    size_t at[3][7];
    for (int k = 0; k < 3; k++)
    {
        const TspClass &c = h->cls[k];
        at[k][0] = take(((size_t)c.tilem + 1) * 4);                                   // tile_ptr
        at[k][1] = take(((size_t)c.tilem + 1) * 4);                                   // panel_row
        at[k][2] = take(((size_t)c.tilenum + 1) * 4);                                 // tile_nnz
        at[k][3] = take(((size_t)c.tilenum * c.BN + 4) * 4);                          // tile_colidx
        at[k][4] = k == 0 ? take((size_t)c.tilenum * tsp_mask_bytes(h->precision) + 16)   // masks
                          : take((size_t)c.tilenum * c.BM * c.BN * vsz + 16);         // dense values
        at[k][5] = k == 0 ? take(((size_t)c.tilenum + 1) * 4) : 0;                    // rec
    }
    if (off > h->tile_block_bytes || off < h->tile_block_bytes / 4)   // reuse what fits, unless it is far too large
    {
        cudaFree(h->tile_block);
        h->tile_block = nullptr; h->tile_block_bytes = 0;
        cudaError_t e = cudaMalloc(&h->tile_block, off);
        if (e != cudaSuccess) { tsp_set_error("tile arrays: cudaMalloc of %zu bytes failed: %s", off, cudaGetErrorString(e)); return TSP_ENOMEM; }
        h->tile_block_bytes = off;
    }
    unsigned char *base = static_cast<unsigned char *>(h->tile_block);
    for (int k = 0; k < 3; k++)
    {
        TspClass &c = h->cls[k];
        c.d_tile_ptr = (int *)(base + at[k][0]);
        c.d_panel_row = (int *)(base + at[k][1]);
        c.d_tile_nnz = (int *)(base + at[k][2]);
        c.d_tile_colidx = (int *)(base + at[k][3]);
        if (k == 0) { c.d_bitmap = base + at[k][4]; c.d_rec = (unsigned int *)(base + at[k][5]); c.d_val = nullptr; }
        else c.d_val = base + at[k][4];
    }
    // zero: everything except the column indices (fully written later); cheaper as a few ranges than as one memset of all
    for (int k = 0; k < 3; k++)
    {
        const size_t from = at[k][0], to = at[k][3];
        TSP_CUDA(cudaMemsetAsync(base + from, 0, to - from, 0));
        const size_t vend = k == 2 ? off : at[k + 1][0];
        TSP_CUDA(cudaMemsetAsync(base + at[k][4], 0, vend - at[k][4], 0));
    }
    return TSP_OK;
}

int tsp_alloc_pack(tsp_handle *h, long long bytes)
{
    const size_t want = (size_t)bytes + 16;
    if (want > h->pack_block_bytes || want < h->pack_block_bytes / 4)
    {
        cudaFree(h->pack_block);
        h->pack_block = nullptr; h->pack_block_bytes = 0;
        cudaError_t e = cudaMalloc(&h->pack_block, want);
        if (e != cudaSuccess) { tsp_set_error("64-row records: cudaMalloc of %lld bytes failed: %s", bytes, cudaGetErrorString(e)); return TSP_ENOMEM; }
        h->pack_block_bytes = want;
    }
    TSP_CUDA(cudaMemsetAsync(h->pack_block, 0, (size_t)bytes + 16, 0));
    h->cls[0].d_pack = static_cast<unsigned char *>(h->pack_block);
    h->cls[0].pack_bytes = bytes;
    return TSP_OK;
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
    void *tmp = nullptr;
    TSP_CUDA(cudaMalloc(&tmp, nelem * vsz));
    cudaError_t e = cudaMemset(tmp, 0, nelem * vsz);
    const int blocks = c.tilenum / 8 + 1 > 148 * 16 ? 148 * 16 : c.tilenum / 8 + 1;
    if (e == cudaSuccess)
    {
        if (h->precision == 0) k_export64<__half><<<blocks, 256>>>(c.tilenum, 0, c.d_rec, c.d_pack, (__half *)tmp);
        else k_export64<float><<<blocks, 256>>>(c.tilenum, 1, c.d_rec, c.d_pack, (float *)tmp);
        e = cudaGetLastError();
    }
    if (e == cudaSuccess) e = cudaMemcpy(h_dst, tmp, nelem * vsz, cudaMemcpyDeviceToHost);
    cudaFree(tmp);
    TSP_CUDA(e);
    return TSP_OK;
}

int tsp_convert_impl(tsp_handle *h, int rowA, int colA, long long nnz64, const int *rowptr_in, const int *colidx_in,
                     const void *val_in, bool csr_on_host, float gamma, float delta, int shard_index, int shard_count)
{
    if (rowA <= 0 || colA <= 0 || nnz64 < 0 || nnz64 > 0x7fffffffLL || shard_count < 1 || shard_index < 0 || shard_index >= shard_count)
    {
        tsp_set_error("convert: bad shape or shard (rowA=%d colA=%d nnz=%lld shard %d/%d)", rowA, colA, nnz64, shard_index, shard_count);
        return TSP_EINVAL;
    }
    TSP_CUDA(cudaSetDevice(h->device));
    TspRange range_all("tsp convert");
    tsp_free_tiles(h);
    h->rowA = rowA; h->colA = colA; h->nnzA = nnz64;
    const int nnz = (int)nnz64;
    const int prec = h->precision;
    const int nb8 = (rowA + 7) / 8;
    const int T = 256;
    const int nchunk = (nb8 + CHAIN_L - 1) / CHAIN_L;
    cudaStream_t st = 0;
    int *pin = nullptr;
    TSP_TRY(pinned(h, &pin));

    // TSP_CONVERT_TRACE=1: wall time of every phase on stderr (each mark waits for the stream, so the total grows a little)
    static const bool trace = getenv("TSP_CONVERT_TRACE") != nullptr;
    struct timeval tv0;
    gettimeofday(&tv0, nullptr);
    auto mark = [&](const char *what) {
        if (!trace) return;
        cudaStreamSynchronize(st);
        struct timeval tv1;
        gettimeofday(&tv1, nullptr);
        fprintf(stderr, "  convert %-28s %8.3f ms\n", what, (tv1.tv_sec - tv0.tv_sec) * 1e3 + (tv1.tv_usec - tv0.tv_usec) * 1e-3);
        tv0 = tv1;
    };

    int fixed = -1;  // src/hetero_split.h:152-169
    if (gamma <= 0.0f) fixed = 0;
    else if (gamma >= 4.0f && delta <= 0.0f) fixed = 1;
    else if (gamma >= 4.0f && delta > 2.0f) fixed = 2;
    const bool want64 = fixed < 0 && gamma < 4.0f;
    const bool want16 = fixed < 0 && (want64 || (delta > 0.0f && !(delta > 2.0f)));

    // ---- workspace: everything whose size follows from nnz and rowA, in one chunk
    const size_t cub_bytes = sort_unique_scratch_bytes(nnz > nb8 + 2 ? nnz : nb8 + 2);
    {
        const size_t n = (size_t)(nnz ? nnz : 1), b = (size_t)nb8 + 16;
        size_t need = 3 * n * 8 + 2 * n * 4 + b * (4 * 9 + 3) + (size_t)nchunk * (8 + 96 + 4 + 12) + b * 8 + cub_bytes + 64 * 256 + (1 << 16);
        if (csr_on_host) need += ((size_t)rowA + 1) * 4 + n * (4 + (prec ? 4 : 2)) + 1024;
        TSP_TRY(reserve_workspace(h, need));
    }
    Workspace ws(h);
    const int *d_rowptr = rowptr_in, *d_colidx = colidx_in;
    const void *d_val = val_in;
    bool values_pending = false, values_in_flight = false;
    struct CopyGuard   // the copy of the values reads caller memory: it must be over on every way out of this function
    {
        tsp_handle *h; bool *active;
        ~CopyGuard() { if (*active) cudaStreamSynchronize(h->side[0]); }
    } copy_guard{h, &values_pending};
    if (csr_on_host)   // upload of the CSR into the workspace
    {
        int *rp, *ci;
        unsigned char *vv;
        const size_t vsz = prec ? 4 : 2;
        TSP_TRY(ws.get(&rp, (size_t)rowA + 1)); TSP_TRY(ws.get(&ci, nnz)); TSP_TRY(ws.get(&vv, (size_t)nnz * vsz));
        TSP_CUDA(cudaMemcpyAsync(rp, rowptr_in, ((size_t)rowA + 1) * 4, cudaMemcpyHostToDevice, st));
        if (nnz) TSP_CUDA(cudaMemcpyAsync(ci, colidx_in, (size_t)nnz * 4, cudaMemcpyHostToDevice, st));
        d_rowptr = rp; d_colidx = ci; d_val = vv;
        values_pending = nnz > 0;   // the values are not needed before stage 5: their upload overlaps the partition kernels
    }
    auto upload_values = [&]() -> int {
        if (!values_pending || values_in_flight) return TSP_OK;
        TSP_CUDA(cudaMemcpyAsync(const_cast<void *>(d_val), val_in, (size_t)nnz * (prec ? 4 : 2), cudaMemcpyHostToDevice, h->side[0]));
        TSP_CUDA(cudaEventRecord(h->join[0], h->side[0]));
        values_in_flight = true;
        return TSP_OK;
    };
    auto wait_values = [&]() -> int {   // orders what is launched on st from here on behind the copy of the values
        if (values_in_flight) TSP_CUDA(cudaStreamWaitEvent(st, h->join[0], 0));
        values_in_flight = false;
        return TSP_OK;
    };
    unsigned long long *keys, *keys_tmp, *keys_col = nullptr, *class_rows_nnz;
    int *u8_ptr, *ucols, *n16, *n64, *entry, *base, *counts, *seq_blk, *seq_idx, *blk_seq, *scalars, *pptr_buf, *pcols_buf, *seq_tiles;
    unsigned char *cls_of, *exit_off, *seq_cls, *cub_tmp;
    double *cost;
    TSP_TRY(ws.get(&keys, nnz)); TSP_TRY(ws.get(&keys_tmp, nnz)); TSP_TRY(ws.get(&u8_ptr, (size_t)nb8 + 9)); TSP_TRY(ws.get(&ucols, nnz));
    TSP_TRY(ws.get(&n16, (size_t)nb8 + 2)); TSP_TRY(ws.get(&n64, (size_t)nb8 + 2)); TSP_TRY(ws.get(&cls_of, nb8));
    TSP_TRY(ws.get(&exit_off, (size_t)nchunk * 8)); TSP_TRY(ws.get(&counts, (size_t)nchunk * 24)); TSP_TRY(ws.get(&entry, nchunk));
    TSP_TRY(ws.get(&base, (size_t)nchunk * 3 + 3));
    TSP_TRY(ws.get(&seq_blk, nb8)); TSP_TRY(ws.get(&seq_cls, nb8)); TSP_TRY(ws.get(&seq_idx, nb8)); TSP_TRY(ws.get(&blk_seq, nb8));
    TSP_TRY(ws.get(&class_rows_nnz, 6)); TSP_TRY(ws.get(&scalars, 64)); TSP_TRY(ws.get(&cub_tmp, cub_bytes));
    TSP_TRY(ws.get(&pptr_buf, (size_t)nb8 + 1)); TSP_TRY(ws.get(&pcols_buf, nnz)); TSP_TRY(ws.get(&seq_tiles, nb8));
    TSP_TRY(ws.get(&cost, nb8));
    if (want16 || want64) TSP_TRY(ws.get(&keys_col, nnz));
    // scalars: [0] distinct (8-row block, column) pairs, [1] CSR check, [2] distinct (panel, column) pairs, [8..17] shard cuts
    int *d_nu = scalars, *d_bad = scalars + 1, *d_np = scalars + 2, *d_cuts = scalars + 8;
    TSP_CUDA(cudaMemsetAsync(scalars, 0, 64 * sizeof(int), st));
    TSP_CUDA(cudaMemsetAsync(class_rows_nnz, 0, 6 * sizeof(unsigned long long), st));

    mark("workspace + upload");
    // ---- stage 1: sorted distinct columns of every 8-row block
    nvtxRangePushA("tsp convert: partition (stages 1-3)");
    {
        const int blocks = blocks_for((long long)rowA * 32, T) > 148 * 64 ? 148 * 64 : blocks_for((long long)rowA * 32, T);
        k_make_block_keys<<<blocks, T, 0, st>>>(rowA, colA, nnz, d_rowptr, d_colidx, keys, d_bad);   // also checks the row pointers of an empty matrix
        TSP_CUDA(cudaGetLastError());
        if (nnz > 0) TSP_TRY(sort_unique_keys(keys, keys_tmp, nnz, 32 + bits_for((unsigned long long)nb8), cub_tmp, cub_bytes, d_nu));
    }
    {
        // the values go up on a side stream while the partition kernels run
        const int rc_up = upload_values();
        if (rc_up != TSP_OK) { nvtxRangePop(); return rc_up; }
    }
    mark("stage 1 keys+sort+unique");
    k_group_offsets<<<blocks_for(nb8 + 9, T), T, 0, st>>>(keys, d_nu, nb8, 8, u8_ptr);   // windows near the end index past nb8
    if (nnz > 0) k_low_words<<<blocks_for(nnz, T) > 148 * 16 ? 148 * 16 : blocks_for(nnz, T), T, 0, st>>>(keys, d_nu, ucols);
    TSP_CUDA(cudaGetLastError());

    // ---- stage 2 + 3: window counts, decisions, chain
    if (want16 || want64)
    {
        // read-back 0 (only when windows are compared at all): the number of pairs, and the CSR check
        TSP_CUDA(cudaMemcpyAsync(pin, scalars, 2 * sizeof(int), cudaMemcpyDeviceToHost, st));
        TSP_CUDA(cudaStreamSynchronize(st));
        if (pin[1])
        {
            nvtxRangePop();
            tsp_set_error("convert: the CSR is inconsistent (row pointers must start at 0, not decrease and end at nnz; columns must lie in [0, %d))", colA);
            return TSP_EINVAL;
        }
        const int pairs = pin[0], bb = bits_for((unsigned long long)nb8);
        TSP_CUDA(cudaMemsetAsync(n16, 0, ((size_t)nb8 + 2) * 4, st)); TSP_CUDA(cudaMemsetAsync(n64, 0, ((size_t)nb8 + 2) * 4, st));
        if (pairs > 0)
        {
            k_col_block_keys<<<blocks_for(pairs, T), T, 0, st>>>(keys, pairs, bb, keys_tmp);
            cub::DoubleBuffer<unsigned long long> db(keys_tmp, keys_col);
            size_t bytes = cub_bytes;
            TSP_CUDA(cub::DeviceRadixSort::SortKeys(cub_tmp, bytes, db, pairs, 0, bb + bits_for((unsigned long long)colA), st));
            k_window_diffs<<<blocks_for(pairs, T), T, 0, st>>>(db.Current(), pairs, bb, want64 ? 1 : 0, n16, n64);
            TSP_CUDA(cudaGetLastError());
            bytes = cub_bytes;
            TSP_CUDA(cub::DeviceScan::InclusiveSum(cub_tmp, bytes, n16, n16, nb8 + 1, st));
            bytes = cub_bytes;
            if (want64) TSP_CUDA(cub::DeviceScan::InclusiveSum(cub_tmp, bytes, n64, n64, nb8 + 1, st));
        }
    }
    mark("stage 2 window counts");
    k_decide<<<blocks_for(nb8, T), T, 0, st>>>(nb8, rowA, gamma, delta, fixed, u8_ptr, n16, n64, cls_of);
    k_chain_local<<<blocks_for((long long)nchunk * 8, 256), 256, 0, st>>>(nb8, nchunk, cls_of, exit_off, counts);
    k_chain_compose<<<1, 1024, 0, st>>>(nchunk, exit_off, counts, entry, base);
    k_chain_emit<<<blocks_for(nchunk, 128), 128, 0, st>>>(nb8, nchunk, rowA, cls_of, entry, base, d_rowptr, seq_blk, seq_cls, seq_idx, blk_seq,
                                                        class_rows_nnz);
    TSP_CUDA(cudaGetLastError());
    // read-back 1: distinct count, CSR check, panels per class, rows and entries per class
    TSP_CUDA(cudaMemcpyAsync(pin, scalars, 2 * sizeof(int), cudaMemcpyDeviceToHost, st));
    TSP_CUDA(cudaMemcpyAsync(pin + 2, base + (size_t)nchunk * 3, 3 * sizeof(int), cudaMemcpyDeviceToHost, st));
    TSP_CUDA(cudaMemcpyAsync(pin + 8, class_rows_nnz, 6 * sizeof(unsigned long long), cudaMemcpyDeviceToHost, st));
    TSP_CUDA(cudaStreamSynchronize(st));
    nvtxRangePop();
    mark("stage 3 decide+chain+readback");
    const int nu = pin[0];
    if (pin[1])
    {
        tsp_set_error("convert: the CSR is inconsistent (row pointers must start at 0, not decrease and end at nnz; columns must lie in [0, %d))", colA);
        return TSP_EINVAL;
    }
    const int totals[3] = {pin[2], pin[3], pin[4]};
    unsigned long long tot_rows_nnz[6];
    memcpy(tot_rows_nnz, pin + 8, sizeof(tot_rows_nnz));
    const int nseq = totals[0] + totals[1] + totals[2];

    // ---- stage 4: sorted distinct columns of every panel
    TspRange range_tiles("tsp convert: tiles (stages 4-6)");
    const int *pptr = nullptr, *pcols = nullptr;
    const bool all8 = totals[0] == 0 && totals[1] == 0;
    if (all8) { pptr = u8_ptr; pcols = ucols; }  // an 8-row panel is one 8-row block
    else
    {
        if (nu)
        {
            k_make_panel_keys<<<blocks_for(nu, T), T, 0, st>>>(keys, nu, blk_seq, keys_tmp);
            TSP_CUDA(cudaGetLastError());
            { unsigned long long *t = keys; keys = keys_tmp; keys_tmp = t; }
            TSP_TRY(sort_unique_keys(keys, keys_tmp, nu, 32 + bits_for((unsigned long long)nseq), cub_tmp, cub_bytes, d_np));
        }
        k_group_offsets<<<blocks_for(nseq + 1, T), T, 0, st>>>(keys, d_np, nseq, 0, pptr_buf);
        if (nu) k_low_words<<<blocks_for(nu, T) > 148 * 16 ? 148 * 16 : blocks_for(nu, T), T, 0, st>>>(keys, d_np, pcols_buf);
        TSP_CUDA(cudaGetLastError());
        pptr = pptr_buf; pcols = pcols_buf;
    }
    if (nseq) k_seq_tiles<<<blocks_for(nseq, T), T, 0, st>>>(nseq, pptr, seq_cls, prec, seq_tiles);
    TSP_CUDA(cudaGetLastError());

    mark("stage 4 panel lists");
    // ---- shard selection: a contiguous range of the panel sequence, balanced by tile bytes (on the device)
    int s0 = 0, s1 = nseq, p0[3] = {0, 0, 0}, p1[3] = {totals[0], totals[1], totals[2]};
    h->row_begin = 0; h->row_end = rowA;
    if (shard_count > 1)
    {
        if (nseq)
        {
            k_panel_costs<<<blocks_for(nseq, T), T, 0, st>>>(nseq, prec, seq_tiles, seq_cls, cost);
            size_t bytes = cub_bytes;
            TSP_CUDA(cub::DeviceScan::InclusiveSum(cub_tmp, bytes, cost, cost, nseq, st));
        }
        k_find_cuts<<<1, 32, 0, st>>>(nseq, rowA, shard_index, shard_count, cost, seq_blk, d_cuts);
        k_shard_bounds<<<blocks_for(nseq ? nseq : 1, T) > 148 * 8 ? 148 * 8 : blocks_for(nseq ? nseq : 1, T), T, 0, st>>>(d_cuts, seq_cls, seq_idx, d_cuts);
        TSP_CUDA(cudaGetLastError());
        // read-back 2 (sharded conversions only): the cuts
        TSP_CUDA(cudaMemcpyAsync(pin, d_cuts, 10 * sizeof(int), cudaMemcpyDeviceToHost, st));
        TSP_CUDA(cudaStreamSynchronize(st));
        s0 = pin[0]; s1 = pin[1];
        for (int k = 0; k < 3; k++)
        {
            p0[k] = pin[2 + k]; p1[k] = pin[5 + k];
            if (p1[k] <= p0[k] || p0[k] == 0x7fffffff) { p0[k] = 0; p1[k] = 0; }
        }
        h->row_begin = pin[8]; h->row_end = pin[9];
        TSP_CUDA(cudaMemsetAsync(class_rows_nnz, 0, 6 * sizeof(unsigned long long), st));
        if (s1 > s0)
        {
            k_class_totals<<<blocks_for(s1 - s0, T) > 148 * 8 ? 148 * 8 : blocks_for(s1 - s0, T), T, 0, st>>>(s0, s1, rowA, seq_cls, seq_blk, d_rowptr,
                                                                                                              class_rows_nnz);
            TSP_CUDA(cudaGetLastError());
        }
    }
    for (int k = 0; k < 3; k++) h->cls[k].tilem = p1[k] - p0[k];

    // ---- tile_ptr: tiles per panel into a workspace array per class, prefix sums; read-back 3: tiles per class
    int *cnt[3], *prow[3], *tptr[3];
    for (int k = 0; k < 3; k++)
    {
        TSP_TRY(ws.get(&cnt[k], (size_t)h->cls[k].tilem + 1)); TSP_TRY(ws.get(&prow[k], (size_t)h->cls[k].tilem + 1));
        TSP_TRY(ws.get(&tptr[k], (size_t)h->cls[k].tilem + 1));
        TSP_CUDA(cudaMemsetAsync(cnt[k], 0, ((size_t)h->cls[k].tilem + 1) * 4, st));
    }
    if (s1 > s0)
    {
        k_class_arrays<<<blocks_for(s1 - s0, T), T, 0, st>>>(s0, s1, seq_tiles, seq_cls, seq_idx, seq_blk, p0[0], p0[1], p0[2], cnt[0], cnt[1], cnt[2],
                                                           prow[0], prow[1], prow[2]);
        TSP_CUDA(cudaGetLastError());
    }
    for (int k = 0; k < 3; k++)
    {
        TspClass &c = h->cls[k];
        size_t bytes = cub_bytes;
        TSP_CUDA(cub::DeviceScan::ExclusiveSum(cub_tmp, bytes, cnt[k], tptr[k], c.tilem + 1, st));
        c.h_tile_ptr.resize((size_t)c.tilem + 1);
        c.h_panel_row.resize(c.tilem);
        TSP_CUDA(cudaMemcpyAsync(c.h_tile_ptr.data(), tptr[k], ((size_t)c.tilem + 1) * 4, cudaMemcpyDeviceToHost, st));
        if (c.tilem) TSP_CUDA(cudaMemcpyAsync(c.h_panel_row.data(), prow[k], (size_t)c.tilem * 4, cudaMemcpyDeviceToHost, st));
    }
    if (shard_count > 1) TSP_CUDA(cudaMemcpyAsync(pin + 8, class_rows_nnz, 6 * sizeof(unsigned long long), cudaMemcpyDeviceToHost, st));
    TSP_CUDA(cudaStreamSynchronize(st));
    if (shard_count > 1) memcpy(tot_rows_nnz, pin + 8, sizeof(tot_rows_nnz));
    for (int k = 0; k < 3; k++)
    {
        TspClass &c = h->cls[k];
        c.tilenum = c.h_tile_ptr[c.tilem];
        c.rows = (int)tot_rows_nnz[k * 2];
        c.nnz = (long long)tot_rows_nnz[k * 2 + 1];
    }

    mark("shards + tile_ptr + readback");
    // ---- the tile arrays of all classes: one allocation
    TSP_TRY(tsp_alloc_tile_arrays(h));
    mark("allocate + clear tile arrays");
    for (int k = 0; k < 3; k++)
    {
        TspClass &c = h->cls[k];
        TSP_CUDA(cudaMemcpyAsync(c.d_tile_ptr, tptr[k], ((size_t)c.tilem + 1) * 4, cudaMemcpyDeviceToDevice, st));
        if (c.tilem) TSP_CUDA(cudaMemcpyAsync(c.d_panel_row, prow[k], (size_t)c.tilem * 4, cudaMemcpyDeviceToDevice, st));
    }
    if (s1 > s0)
    {
        const int blocks = blocks_for((long long)(s1 - s0) * 32, T) > 148 * 32 ? 148 * 32 : blocks_for((long long)(s1 - s0) * 32, T);
        k_fill_colidx<<<blocks, T, 0, st>>>(s0, s1, prec, pptr, pcols, seq_cls, seq_idx, p0[0], p0[1], p0[2], h->cls[0].d_tile_ptr,
                                            h->cls[1].d_tile_ptr, h->cls[2].d_tile_ptr, h->cls[0].d_tile_colidx, h->cls[1].d_tile_colidx,
                                            h->cls[2].d_tile_colidx);
        TSP_CUDA(cudaGetLastError());
        // ---- stage 5
        TSP_TRY(wait_values());
        const int vblocks = blocks_for((long long)rowA * 32, T) > 148 * 64 ? 148 * 64 : blocks_for((long long)rowA * 32, T);
        if (prec == 0)
            k_place_values<__half><<<vblocks, T, 0, st>>>(rowA, 0, s0, s1, d_rowptr, d_colidx, (const __half *)d_val, blk_seq, seq_cls, seq_idx,
                                                          seq_blk, pptr, pcols, p0[0], p0[1], p0[2], h->cls[0].d_tile_ptr, h->cls[1].d_tile_ptr,
                                                          h->cls[2].d_tile_ptr, h->cls[0].d_tile_nnz, h->cls[1].d_tile_nnz, h->cls[2].d_tile_nnz,
                                                          (unsigned int *)h->cls[0].d_bitmap, (__half *)h->cls[1].d_val, (__half *)h->cls[2].d_val);
        else
            k_place_values<float><<<vblocks, T, 0, st>>>(rowA, 1, s0, s1, d_rowptr, d_colidx, (const float *)d_val, blk_seq, seq_cls, seq_idx,
                                                         seq_blk, pptr, pcols, p0[0], p0[1], p0[2], h->cls[0].d_tile_ptr, h->cls[1].d_tile_ptr,
                                                         h->cls[2].d_tile_ptr, h->cls[0].d_tile_nnz, h->cls[1].d_tile_nnz, h->cls[2].d_tile_nnz,
                                                         (unsigned int *)h->cls[0].d_bitmap, (float *)h->cls[1].d_val, (float *)h->cls[2].d_val);
        TSP_CUDA(cudaGetLastError());
    }
    mark("stage 5 colidx + values");
    for (int k = 0; k < 3; k++)  // tile_nnz: exclusive scan over tilenum+1 entries (src/csr2tile.h:786)
    {
        TspClass &c = h->cls[k];
        size_t bytes = 0;
        TSP_CUDA(cub::DeviceScan::ExclusiveSum(nullptr, bytes, c.d_tile_nnz, c.d_tile_nnz, c.tilenum + 1, st));
        void *tmp = cub_tmp;
        if (bytes > cub_bytes) { unsigned char *more; TSP_TRY(ws.get(&more, bytes)); tmp = more; }
        TSP_CUDA(cub::DeviceScan::ExclusiveSum(tmp, bytes, c.d_tile_nnz, c.d_tile_nnz, c.tilenum + 1, st));
    }

    // ---- stage 6: records of the 64-row class
    {
        TspClass &c = h->cls[0];
        c.d_pack = nullptr; c.pack_bytes = 0;
        if (c.tilenum > 0)
        {
            unsigned int *units, *prefix;
            unsigned char *dense;
            unsigned short *row_off;
            TSP_TRY(ws.get(&units, (size_t)c.tilenum + 1)); TSP_TRY(ws.get(&prefix, (size_t)c.tilenum + 1)); TSP_TRY(ws.get(&dense, c.tilenum));
            TSP_TRY(ws.get(&row_off, (size_t)c.tilenum * 64));
            TSP_CUDA(cudaMemsetAsync(units + c.tilenum, 0, 4, st));
            const int wblocks = blocks_for((long long)c.tilenum * 32, T) > 148 * 32 ? 148 * 32 : blocks_for((long long)c.tilenum * 32, T);
            k_rec_sizes<<<wblocks, T, 0, st>>>(c.tilenum, prec, (const unsigned int *)c.d_bitmap, units, dense, row_off);
            size_t bytes = 0;
            TSP_CUDA(cub::DeviceScan::ExclusiveSum(nullptr, bytes, units, prefix, c.tilenum + 1, st));
            void *tmp = cub_tmp;
            if (bytes > cub_bytes) { unsigned char *more; TSP_TRY(ws.get(&more, bytes)); tmp = more; }
            TSP_CUDA(cub::DeviceScan::ExclusiveSum(tmp, bytes, units, prefix, c.tilenum + 1, st));
            k_rec_finish<<<blocks_for(c.tilenum + 1, T), T, 0, st>>>(c.tilenum, prefix, dense, c.d_rec);
            TSP_CUDA(cudaGetLastError());
            // read-back 4 (only when there are 64-row tiles): bytes of all records
            TSP_CUDA(cudaMemcpyAsync(pin, prefix + c.tilenum, 4, cudaMemcpyDeviceToHost, st));
            TSP_CUDA(cudaStreamSynchronize(st));
            const long long total_units = (unsigned int)pin[0];
            if (total_units >= 0x7fffffffLL) { tsp_set_error("convert: the 64-row tile records exceed 32 GB"); return TSP_EINVAL; }
            TSP_TRY(tsp_alloc_pack(h, total_units * 16));
            k_init_positions<<<c.tilenum > 148 * 16 ? 148 * 16 : c.tilenum, 64, 0, st>>>(c.tilenum, prec, c.d_rec, c.d_pack);
            const int vblocks = blocks_for((long long)rowA * 32, T) > 148 * 64 ? 148 * 64 : blocks_for((long long)rowA * 32, T);
            if (prec == 0)
                k_place_values64<__half><<<vblocks, T, 0, st>>>(rowA, 0, s0, s1, d_rowptr, d_colidx, (const __half *)d_val, blk_seq, seq_cls, seq_idx,
                                                                seq_blk, pptr, pcols, p0[0], c.d_tile_ptr, (const unsigned int *)c.d_bitmap, row_off,
                                                                c.d_rec, (__half *)c.d_pack);
            else
                k_place_values64<float><<<vblocks, T, 0, st>>>(rowA, 1, s0, s1, d_rowptr, d_colidx, (const float *)d_val, blk_seq, seq_cls, seq_idx,
                                                               seq_blk, pptr, pcols, p0[0], c.d_tile_ptr, (const unsigned int *)c.d_bitmap, row_off,
                                                               c.d_rec, (float *)c.d_pack);
            TSP_CUDA(cudaGetLastError());
        }
    }
    TSP_CUDA(cudaStreamSynchronize(st));
    mark("stage 6 records");
    // a large workspace (hundreds of millions of entries) is given back; a small one stays for the next conversion
    size_t held = 0;
    for (auto &ch : h->ws_chunks) held += ch.second;
    if (held > ((size_t)2 << 30)) tsp_free_workspace(h);
    h->converted = true;
    return TSP_OK;
}
