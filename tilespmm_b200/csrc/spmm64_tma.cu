// SpMM kernel for the 64-row tile class, TMA + tcgen05 form (sm_100a).  Selected with TSP_SPMM64=tma; the default is
// the form in spmm64.cu whose producer warps gather with cp.async, because it is faster on B200: 0.207 ms vs 0.242 ms
// on the 27-point stencil (TF32, 128 columns), 0.558 vs 0.726 ms on the mixed-density matrix (TF32, 256 columns),
// 0.237 vs 0.281 ms on R-MAT scale 18 (FP16, 64 columns) -- a gather4 request moves only 4 x 128 bytes.
//
// Replaces upstream stir_spmm_cuda_kernel_v64* (src/tilespmm_cuda.h:1025-1632) and switch_tilespmm_cuda_v64
// (src/tilespmm_cuda.h:1710-1744).  One CTA owns one task (a 64-row panel or a slice of a split panel) and one column
// stripe of up to 256 columns.  Roles:
//   warp 0     one lane is the producer.  Per tile it reads the tile's column indices (16-byte loads), arms the
//              slot's mbarrier with the byte count and issues (a) one cp.async.bulk for the 4 KB A tile, which the
//              conversion stores in the K-major core-matrix order tcgen05.mma reads, and (b) one
//              cp.async.bulk.tensor.2d ... tile::gather4 per four gathered B rows and 128-byte column block: the copy
//              engine fetches the four rows named by the indices and writes them in the swizzled MN-major operand
//              layout (FP16: 128-byte swizzle, or 64-byte swizzle for 64-byte rows; TF32: 128-byte swizzle with
//              32-byte atoms, the only MN-major mode for 32-bit operands).  No thread touches the data.
//   warp 1     allocates tensor memory; one lane issues two tcgen05.mma (M=64, N=stripe, K=16 FP16 / K=8 TF32) per
//              tile and releases ring slots with tcgen05.commit.
//   warps 2-5  epilogue: tcgen05.ld of the 64 x N FP32 accumulator (kept in tensor memory for the whole task) -> C,
//              16-byte stores, or vector red.global.add for the slices of a split panel.
// Every mbarrier wait is bounded; when one runs out the kernel records it in *err, and returns after freeing
// tensor memory.
#include <cuda.h>

#include "tsp_internal.cuh"

namespace
{

constexpr unsigned WAIT_LIMIT = 1u << 22;
constexpr int THREADS = 6 * 32;

template <int PREC, int N>
struct CfgT
{
    static constexpr int SZ = PREC == 0 ? 2 : 4;
    static constexpr int BNK = PREC == 0 ? 32 : 16;           // K extent of a tile = gathered rows per tile
    static constexpr int A_BYTES = 64 * BNK * SZ;             // 4096
    static constexpr int RB = N * SZ;                         // bytes of one gathered row segment
    static constexpr int BOX_BYTES = RB >= 128 ? 128 : 64;    // inner extent of one gather4 box
    static constexpr int BOX_COLS = BOX_BYTES / SZ;
    static constexpr int NBOX = RB / BOX_BYTES;               // column boxes per row
    static constexpr int B_BYTES = BNK * RB;
    static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
    static constexpr int STAGES = N == 256 ? 4 : (N == 128 ? 4 : (N == 64 ? 6 : 8));
    static constexpr int SMEM = STAGES * STAGE_BYTES + 1024;  // + slack to align the ring to 1 KB
    // swizzle / layout-type field of the tcgen05 shared-memory descriptor and atom geometry (see the cp.async form)
    static constexpr int MODE = PREC == 1 ? 1 : (RB >= 128 ? 2 : 4);
    static constexpr int ATOM_ROWS = PREC == 1 ? 4 : 8;
    static constexpr int ATOM_BYTES = ATOM_ROWS * BOX_BYTES;
    static constexpr int KATOMS = BNK / ATOM_ROWS;
    static constexpr int KATOMS_PER_MMA = 2;
    static constexpr int TMEM_COLS = N < 32 ? 32 : N;
};

__device__ __forceinline__ unsigned smem_u32(const void *p) { return (unsigned)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(unsigned bar, unsigned count) { asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(bar), "r"(count)); }
__device__ __forceinline__ void mbar_expect_tx(unsigned bar, unsigned bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_wait(unsigned bar, unsigned parity)
{
    for (unsigned it = 0; it < WAIT_LIMIT; it++)
    {
        unsigned done;
        asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}\n"
                     : "=r"(done) : "r"(bar), "r"(parity) : "memory");
        if (done) return true;
    }
    return false;
}
__device__ __forceinline__ void bulk_g2s(unsigned dst, const void *src, unsigned bytes, unsigned bar)
{
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}
// four rows (r0..r3) of the 2-D tensor, columns x .. x + box, into 4 x box bytes of shared memory
__device__ __forceinline__ void tma_gather4(unsigned dst, const CUtensorMap *map, int x, int r0, int r1, int r2, int r3, unsigned bar)
{
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile::gather4.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6, %7}], [%2];\n"
                 ::"r"(dst), "l"(map), "r"(bar), "r"(x), "r"(r0), "r"(r1), "r"(r2), "r"(r3) : "memory");
}
__device__ __forceinline__ unsigned long long make_desc(unsigned addr, unsigned lbo_bytes, unsigned sbo_bytes, unsigned layout_type)
{
    unsigned long long d = 0;
    d |= (unsigned long long)((addr >> 4) & 0x3fff);
    d |= (unsigned long long)((lbo_bytes >> 4) & 0x3fff) << 16;
    d |= (unsigned long long)((sbo_bytes >> 4) & 0x3fff) << 32;
    d |= 1ull << 46;
    d |= (unsigned long long)layout_type << 61;
    return d;
}
template <int PREC>
__device__ __forceinline__ void umma(unsigned tmem_d, unsigned long long da, unsigned long long db, unsigned idesc, unsigned accumulate)
{
    if constexpr (PREC == 0)
        asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}\n"
                     ::"r"(tmem_d), "l"(da), "l"(db), "r"(idesc), "r"(accumulate) : "memory");
    else
        asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}\n"
                     ::"r"(tmem_d), "l"(da), "l"(db), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(unsigned bar)
{
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_ld32(unsigned taddr, unsigned (&r)[32])
{
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                 "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
                   "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]),
                   "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
                   "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
                 : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
}

template <int PREC, int N>
__global__ void __launch_bounds__(THREADS)
k_spmm64_tma(const __grid_constant__ CUtensorMap bmap, int ntasks, int ldb, int row_begin, const unsigned int *__restrict__ task_row,
             const int *__restrict__ task_start, const int *__restrict__ tile_colidx, const unsigned char *__restrict__ tile_val,
             float *__restrict__ dC, int *__restrict__ err)
{
    using C = CfgT<PREC, N>;
    constexpr int S = C::STAGES;
    extern __shared__ unsigned char smem_raw[];
    __shared__ __align__(8) unsigned long long bars[2 * C::STAGES + 1];
    __shared__ unsigned tmem_slot;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, tid = threadIdx.x;
    const int task = blockIdx.x, stripe = blockIdx.y;
    const unsigned ring = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const unsigned bar_full = smem_u32(&bars[0]), bar_empty = smem_u32(&bars[S]), bar_done = smem_u32(&bars[2 * S]);

    const unsigned int trow = task_row[task];
    const bool split = (trow >> 31) != 0;
    const int first_row = (int)(trow & 0x7fffffffu) - row_begin;
    const int t0 = task_start[task], nt = task_start[task + 1] - t0;

    if (tid == 0)
    {
        for (int s = 0; s < S; s++) { mbar_init(bar_full + 8 * s, 1); mbar_init(bar_empty + 8 * s, 1); }
        mbar_init(bar_done, 1);
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    if (warp == 1)
    {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_u32(&tmem_slot)), "r"(C::TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
    const unsigned tmem_base = tmem_slot;
    bool ok = true;

    if (warp == 0)
    {
        // ------------------------------------------------------------ producer: one lane drives the copy engine
        // (spreading the requests over the lanes of the warp measured slower: 0.283 ms vs 0.242 ms on the stencil)
        if (lane == 0)
        {
            const int x0 = stripe * N;
            const int4 *idx = reinterpret_cast<const int4 *>(tile_colidx + (size_t)t0 * C::BNK);   // BNK/4 groups of four rows per tile
            const unsigned char *a_src = tile_val + (size_t)t0 * C::A_BYTES;
            int4 rows[C::BNK / 4];
            if (nt > 0)
            {
#pragma unroll
                for (int g = 0; g < C::BNK / 4; g++) rows[g] = __ldg(idx + g);
            }
            for (int i = 0; i < nt; i++)
            {
                const int s = i % S;
                if (i >= S && !mbar_wait(bar_empty + 8 * s, ((i / S) - 1) & 1)) { ok = false; break; }
                const unsigned st = ring + s * C::STAGE_BYTES, bar = bar_full + 8 * s;
                mbar_expect_tx(bar, C::STAGE_BYTES);
                bulk_g2s(st, a_src, C::A_BYTES, bar);
                a_src += C::A_BYTES;
#pragma unroll
                for (int g = 0; g < C::BNK / 4; g++)
                {
                    // rows 4g .. 4g+3 of the tile; for FP16 two groups share one 8-row atom
                    const unsigned atom = (unsigned)((g * 4) / C::ATOM_ROWS) * C::ATOM_BYTES + (unsigned)((g * 4) % C::ATOM_ROWS) * C::BOX_BYTES;
#pragma unroll
                    for (int b = 0; b < C::NBOX; b++)
                        tma_gather4(st + C::A_BYTES + (unsigned)b * C::KATOMS * C::ATOM_BYTES + atom, &bmap, x0 + b * C::BOX_COLS,
                                    rows[g].x, rows[g].y, rows[g].z, rows[g].w, bar);
                }
                if (i + 1 < nt)
                {
                    idx += C::BNK / 4;
#pragma unroll
                    for (int g = 0; g < C::BNK / 4; g++) rows[g] = __ldg(idx + g);
                }
            }
        }
    }
    else if (warp == 1)
    {
        // ------------------------------------------------------------ MMA issuer
        if (lane == 0)
        {
            // instruction descriptor: D = F32, A/B = F16 or TF32, A K-major, B MN-major, N/8, M/16
            const unsigned fmt = PREC == 0 ? 0u : 2u;
            const unsigned idesc = (1u << 4) | (fmt << 7) | (fmt << 10) | (0u << 15) | (1u << 16) | ((unsigned)(N >> 3) << 17) | ((64u >> 4) << 24);
            for (int i = 0; i < nt && ok; i++)
            {
                const int s = i % S;
                ok = mbar_wait(bar_full + 8 * s, (i / S) & 1);
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
                const unsigned st = ring + s * C::STAGE_BYTES;
#pragma unroll
                for (int kk = 0; kk < 2; kk++)
                {
                    // A: K-major, no swizzle; the two core-matrix columns of this K step are 1 KB apart, 8-row groups 128 B apart
                    const unsigned long long da = make_desc(st + kk * 2048, 1024, 128, 0);
                    // B: MN-major; column atoms KATOMS*ATOM_BYTES apart, K atoms ATOM_BYTES apart
                    const unsigned long long db = make_desc(st + C::A_BYTES + kk * C::KATOMS_PER_MMA * C::ATOM_BYTES,
                                                            C::KATOMS * C::ATOM_BYTES, C::ATOM_BYTES, (unsigned)C::MODE);
                    umma<PREC>(tmem_base, da, db, idesc, (i > 0 || kk > 0) ? 1u : 0u);
                }
                umma_commit(bar_empty + 8 * s);  // frees the slot when these MMAs have read it
            }
            if (ok && nt > 0) umma_commit(bar_done);
        }
    }
    else
    {
        // ------------------------------------------------------------ epilogue (warps 2-5: tensor-memory quarter = warp % 4)
        if (nt > 0)
        {
            ok = __all_sync(0xffffffffu, mbar_wait(bar_done, 0));
            asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
        }
        if (ok)
        {
            // with M = 64 the accumulator row r lives in tensor-memory lane (r/16)*32 + r%16
            const int quarter = warp & 3;
            const int row = quarter * 16 + (lane & 15);
            float *crow = dC + (size_t)(first_row + row) * (size_t)ldb + (size_t)stripe * N;
#pragma unroll 1
            for (int c0 = 0; c0 < N; c0 += 32)
            {
                unsigned r[32];
                if (nt > 0) tmem_ld32(tmem_base + ((unsigned)(quarter * 32) << 16) + (unsigned)c0, r);
                else
                {
#pragma unroll
                    for (int j = 0; j < 32; j++) r[j] = 0u;
                }
                if (lane < 16)
                {
#pragma unroll
                    for (int j = 0; j < 32; j += 4)
                    {
                        if (split)
                            asm volatile("red.global.add.v4.f32 [%0], {%1,%2,%3,%4};\n" ::"l"(crow + c0 + j), "f"(__uint_as_float(r[j])),
                                         "f"(__uint_as_float(r[j + 1])), "f"(__uint_as_float(r[j + 2])), "f"(__uint_as_float(r[j + 3])) : "memory");
                        else
                            *reinterpret_cast<uint4 *>(crow + c0 + j) = make_uint4(r[j], r[j + 1], r[j + 2], r[j + 3]);
                    }
                }
            }
        }
    }
    if (!ok) atomicExch(err, 1);
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    if (warp == 1)
    {
        asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"(C::TMEM_COLS) : "memory");
    }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                                  const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// Tensor map over B (colA rows x colB columns, row-major) for gather4: the box is {BOX_COLS, 1}; the instruction names
// four rows and one column offset.
int make_b_map(CUtensorMap *map, int precision, const void *d_b, int colA, int colB, int box_cols, int box_bytes)
{
    static EncodeTiledFn encode = nullptr;
    if (!encode)
    {
        void *fn = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess || !fn)
        {
            tsp_set_error("spmm64: cuTensorMapEncodeTiled is not available from this driver");
            return TSP_ECUDA;
        }
        encode = (EncodeTiledFn)fn;
    }
    const cuuint64_t dims[2] = {(cuuint64_t)colB, (cuuint64_t)colA};
    const cuuint64_t strides[1] = {(cuuint64_t)colB * (precision ? 4 : 2)};
    const cuuint32_t box[2] = {(cuuint32_t)box_cols, 1};
    const cuuint32_t estr[2] = {1, 1};
    const CUtensorMapSwizzle sw = precision ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B : (box_bytes >= 128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B);
    const CUresult r = encode(map, precision ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void *>(d_b), dims,
                              strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, sw, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) { tsp_set_error("spmm64: cuTensorMapEncodeTiled failed with %d (B must be 16-byte aligned)", (int)r); return TSP_ECUDA; }
    return TSP_OK;
}

template <int PREC, int N>
int launch64(tsp_handle *h, const void *d_b, float *d_c, int colB, cudaStream_t s)
{
    using C = CfgT<PREC, N>;
    TspClass &c = h->cls[0];
    static bool configured[8] = {false};
    auto kern = k_spmm64_tma<PREC, N>;
    if (!configured[h->device & 7])
    {
        TSP_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM));
        configured[h->device & 7] = true;
    }
    if (c.ntasks == 0) return TSP_OK;
    if (h->bmap_ptr != d_b || h->bmap_cols != colB || h->bmap_box != C::BOX_COLS)   // the map depends on B's address and shape only
    {
        TSP_TRY(make_b_map(reinterpret_cast<CUtensorMap *>(h->bmap), PREC, d_b, h->colA, colB, C::BOX_COLS, C::BOX_BYTES));
        h->bmap_ptr = d_b; h->bmap_cols = colB; h->bmap_box = C::BOX_COLS;
    }
    dim3 grid(c.ntasks, colB / N);
    kern<<<grid, THREADS, C::SMEM, s>>>(*reinterpret_cast<const CUtensorMap *>(h->bmap), c.ntasks, colB, h->row_begin, c.d_task_row, c.d_task_start,
                                       c.d_tile_colidx, (const unsigned char *)c.d_val, d_c, h->d_error);
    TSP_CUDA(cudaGetLastError());
    h->launches++;
    return TSP_OK;
}

template <int PREC>
int launch64_width(tsp_handle *h, const void *d_b, float *d_c, int colB, cudaStream_t s)
{
    switch (tsp_stripe_width(0, colB))
    {
    case 32: return launch64<PREC, 32>(h, d_b, d_c, colB, s);
    case 256: return launch64<PREC, 256>(h, d_b, d_c, colB, s);
    case 128: return launch64<PREC, 128>(h, d_b, d_c, colB, s);
    default: return launch64<PREC, 64>(h, d_b, d_c, colB, s);
    }
}

}  // namespace

int tsp_launch_class64_tma(tsp_handle *h, const void *d_b, float *d_c, int colB, cudaStream_t s)
{
    return h->precision == 0 ? launch64_width<0>(h, d_b, d_c, colB, s) : launch64_width<1>(h, d_b, d_c, colB, s);
}
