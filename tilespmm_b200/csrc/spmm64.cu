// SpMM kernel for the 64-row tile class: tcgen05.mma with the accumulator in tensor memory (sm_100a).
//
// Replaces upstream stir_spmm_cuda_kernel_v64* (src/tilespmm_cuda.h:1025-1632) and switch_tilespmm_cuda_v64
// (src/tilespmm_cuda.h:1710-1744).  One CTA owns one task (a 64-row panel or a slice of a split panel) and one
// column stripe of up to 256 columns, so the A tiles and column indices are read once per 256 columns
// (upstream: once per 64).  Roles:
//   warps 0-3  producers: gather the B rows named by tile_colidx with 16-byte cp.async into a STAGES-deep ring,
//              writing the swizzled MN-major operand layout tcgen05.mma reads, plus the A tile, which
//              the conversion already stores in the K-major core-matrix order (one 4 KB cp.async.bulk per tile);
//              afterwards they are the epilogue: tcgen05.ld of the 64 x N FP32 accumulator -> C.
//   warp 4     allocates tensor memory; one elected lane issues two tcgen05.mma (M=64, N=stripe, K=16 FP16 /
//              K=8 TF32) per tile and releases ring slots with tcgen05.commit.
// The accumulator of a whole task stays in tensor memory (64 lanes x N columns) and is written once, with
// vector stores, or vector red.global.add for the slices of a split panel.
// Every wait on an mbarrier is bounded; when one runs out the kernel records it in *err and returns.
#include "tsp_internal.cuh"

namespace
{

constexpr unsigned WAIT_LIMIT = 1u << 22;

template <int PREC, int N>
struct Cfg64
{
    static constexpr int PW = N >= 128 ? 8 : 4;               // producer (and epilogue) warps
    static constexpr int THREADS = (PW + 1) * 32;
    static constexpr int SZ = PREC == 0 ? 2 : 4;
    static constexpr int BNK = PREC == 0 ? 32 : 16;           // K extent of a tile
    static constexpr int A_BYTES = 64 * BNK * SZ;             // 4096
    static constexpr int RB = N * SZ;                         // bytes of one gathered row segment
    static constexpr int CPR = RB / 16;
    static constexpr int B_BYTES = BNK * RB;
    static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
    // ring depth and how many tiles the producers run ahead of what they have published: a slot is reused
    // STAGES tiles later, LAG+1 tiles are in flight to memory, and the MMA has STAGES-LAG tiles of slack
    static constexpr int STAGES = N >= 128 ? 4 : (N == 64 ? 6 : 8);
    static constexpr int LAG = N >= 128 ? 2 : 4;
    static constexpr int SMEM = STAGES * STAGE_BYTES + 1024;  // + slack to align the ring to 1 KB
    // Shared-memory layout of the gathered rows (the MN-major B operand):
    //   FP16, rows >= 128 B : 128-byte swizzle, atoms of 8 K-rows x 128 B, 16-byte chunks XORed with the row
    //   FP16, 64-byte rows  : 64-byte swizzle, atoms of 8 K-rows x 64 B
    //   TF32                : the only MN-major mode for 32-bit operands, "128-byte swizzle with 32-byte
    //                         atomicity": atoms of 4 K-rows x 128 B, 32-byte chunks XORed with the row
    static constexpr int MODE = PREC == 1 ? 1 : (RB >= 128 ? 2 : 4);   // layout-type field of the descriptor
    static constexpr int ATOM_ROWS = PREC == 1 ? 4 : 8;
    static constexpr int ATOM_BYTES = ATOM_ROWS * (RB >= 128 ? 128 : 64);
    static constexpr int KATOMS = BNK / ATOM_ROWS;            // atoms along K per tile (4)
    static constexpr int KATOMS_PER_MMA = 2;                  // K = 16 halves = 2x8 rows / 8 floats = 2x4 rows
    static constexpr int TMEM_COLS = N < 32 ? 32 : N;
    static constexpr int B_ITERS = (BNK * CPR) / (PW * 32);
    static constexpr int A_ITERS = A_BYTES / 16 / (PW * 32);
    static constexpr int KPI = PW * 32 / CPR;                 // tile rows covered by one CTA-wide copy
};

__device__ __forceinline__ unsigned smem_u32(const void *p) { return (unsigned)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void cp_async16(unsigned smem, const void *gmem)
{
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(smem), "l"(gmem));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int K>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(K) : "memory"); }

__device__ __forceinline__ void mbar_init(unsigned bar, unsigned count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_arrive(unsigned bar)
{
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(unsigned bar, unsigned bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(bar), "r"(bytes) : "memory");
}
// one bulk copy (the copy engine, no per-thread work): global -> shared, completion counted in bytes on the mbarrier
__device__ __forceinline__ void bulk_g2s(unsigned dst, const void *src, unsigned bytes, unsigned bar)
{
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}
// bounded wait: false when the phase did not complete within WAIT_LIMIT polls
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

__device__ __forceinline__ unsigned long long make_desc(unsigned addr, unsigned lbo_bytes, unsigned sbo_bytes, unsigned layout_type)
{
    // shared-memory matrix descriptor of tcgen05.mma: start address, leading and stride byte offsets
    // (all in 16-byte units), descriptor version 1, swizzle mode in bits 61-63
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
__global__ void __launch_bounds__(Cfg64<PREC, N>::THREADS)
k_spmm64(int ntasks, int ldb, int row_begin, const unsigned int *__restrict__ task_row, const int *__restrict__ task_start,
         const int *__restrict__ tile_colidx, const unsigned char *__restrict__ tile_val, const unsigned char *__restrict__ dB,
         float *__restrict__ dC, int *__restrict__ err)
{
    using C = Cfg64<PREC, N>;
    constexpr int S = C::STAGES, PRODUCER_WARPS = C::PW;
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
        for (int s = 0; s < S; s++) { mbar_init(bar_full + 8 * s, PRODUCER_WARPS + 1); mbar_init(bar_empty + 8 * s, 1); }
        mbar_init(bar_done, 1);
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    if (warp == PRODUCER_WARPS)
    {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_u32(&tmem_slot)), "r"(C::TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
    const unsigned tmem_base = tmem_slot;
    bool ok = true;

    if (warp < PRODUCER_WARPS)
    {
        // ------------------------------------------------------------ producers
        // Chunk q = it*PW*32 + tid of a tile is 16-byte chunk c = tid % CPR of row k = it*KPI + tid/CPR, so the
        // source column offset and the swizzled destination of every copy are loop invariants.
        const unsigned ldb_b = (unsigned)ldb * C::SZ;
        const int c_mine = tid % C::CPR, k_mine = tid / C::CPR;
        const unsigned char *gsrc = dB + (size_t)stripe * C::RB + (size_t)c_mine * 16;
        const int *idx_ptr = tile_colidx + (size_t)t0 * C::BNK + k_mine;
        const unsigned char *a_src = tile_val + (size_t)t0 * C::A_BYTES;
        int cols_next[C::B_ITERS];
        unsigned dst_off[C::B_ITERS];
#pragma unroll
        for (int it = 0; it < C::B_ITERS; it++)
        {
            const int k = it * C::KPI + k_mine, c = c_mine;
            if (C::MODE == 2) { const int ka = k >> 3, kr = k & 7; dst_off[it] = ((c >> 3) * C::KATOMS + ka) * 1024 + kr * 128 + (((c & 7) ^ kr) << 4); }
            else if (C::MODE == 4) { const int ka = k >> 3, kr = k & 7; dst_off[it] = ka * 512 + kr * 64 + ((c ^ ((kr >> 1) & 3)) << 4); }
            else { const int ka = k >> 2, kr = k & 3; dst_off[it] = ((c >> 3) * C::KATOMS + ka) * 512 + kr * 128 + (((((c & 7) >> 1) ^ kr) << 5) | ((c & 1) << 4)); }
            dst_off[it] += C::A_BYTES;
            cols_next[it] = nt > 0 ? __ldg(idx_ptr + it * C::KPI) : 0;
        }
        auto publish = [&](int i) {  // tile i is complete in shared memory: hand it to the MMA warp
            asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_full + 8 * (i % S));
        };
        int published = 0;
        for (int i = 0; i < nt && ok; i++)
        {
            const int s = i % S;
            if (i >= S) ok = __all_sync(0xffffffffu, mbar_wait(bar_empty + 8 * s, ((i / S) - 1) & 1));  // warp-uniform outcome
            if (!ok) break;
            const unsigned st = ring + s * C::STAGE_BYTES;
            // the A tile is already in operand order in global memory: one 4 KB bulk copy, whose bytes are
            // counted on the slot's full barrier together with the producer warps' arrivals
            if (tid == 0)
            {
                mbar_expect_tx(bar_full + 8 * s, C::A_BYTES);
                bulk_g2s(st, a_src, C::A_BYTES, bar_full + 8 * s);
            }
            a_src += C::A_BYTES;
#pragma unroll
            for (int it = 0; it < C::B_ITERS; it++)
                cp_async16(st + dst_off[it], gsrc + (unsigned long long)(unsigned)cols_next[it] * ldb_b);
            cp_async_commit();
            idx_ptr += C::BNK;
            if (i + 1 < nt)
            {
#pragma unroll
                for (int it = 0; it < C::B_ITERS; it++) cols_next[it] = __ldg(idx_ptr + it * C::KPI);
            }
            if (i >= C::LAG)
            {
                cp_async_wait<C::LAG>();  // the group of tile i-LAG has landed
                publish(i - C::LAG);
                published = i - C::LAG + 1;
            }
        }
        cp_async_wait<0>();
        if (ok)
            for (int i = published; i < nt; i++) publish(i);

        // ------------------------------------------------------------ epilogue
        if (ok && nt > 0)
        {
            ok = __all_sync(0xffffffffu, mbar_wait(bar_done, 0));
            asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
        }
        if (ok)
        {
            // with M = 64 the accumulator row r lives in tensor-memory lane (r/16)*32 + r%16
            // a warp reads the 32 lanes of its quarter (warp % 4); with 8 epilogue warps each quarter is shared
            // by two warps that take one half of the columns each
            const int quarter = warp & 3, part = warp >> 2;
            constexpr int COLS_PER_WARP = N / (PRODUCER_WARPS / 4);
            const int row = quarter * 16 + (lane & 15);
            float *crow = dC + (size_t)(first_row + row) * (size_t)ldb + (size_t)stripe * N;
#pragma unroll 1
            for (int c0 = part * COLS_PER_WARP; c0 < (part + 1) * COLS_PER_WARP; c0 += 32)
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
    else if (lane == 0)
    {
        // ------------------------------------------------------------ MMA issuer
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
                // A: K-major, no swizzle; the two core-matrix columns of this K step are 1 KB apart,
                // 8-row groups 128 B apart
                const unsigned long long da = make_desc(st + kk * 2048, 1024, 128, 0);
                // B: MN-major; 64-column (128-byte) atoms KATOMS KB apart, K atoms ATOM_BYTES apart
                const unsigned long long db = make_desc(st + C::A_BYTES + kk * C::KATOMS_PER_MMA * C::ATOM_BYTES,
                                                        C::KATOMS * C::ATOM_BYTES, C::ATOM_BYTES, (unsigned)C::MODE);
                umma<PREC>(tmem_base, da, db, idesc, (i > 0 || kk > 0) ? 1u : 0u);
            }
            umma_commit(bar_empty + 8 * s);  // frees the slot when these MMAs have read it
        }
        if (ok && nt > 0) umma_commit(bar_done);
    }
    if (!ok) atomicExch(err, 1);
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    if (warp == PRODUCER_WARPS)
    {
        asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"(C::TMEM_COLS) : "memory");
    }
}

template <int PREC, int N>
int launch64(tsp_handle *h, const void *d_b, float *d_c, int colB, cudaStream_t s)
{
    using C = Cfg64<PREC, N>;
    TspClass &c = h->cls[0];
    static bool configured[8] = {false};
    auto kern = k_spmm64<PREC, N>;
    if (!configured[h->device & 7])
    {
        TSP_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM));
        configured[h->device & 7] = true;
    }
    if (c.ntasks == 0) return TSP_OK;
    dim3 grid(c.ntasks, colB / N);
    kern<<<grid, C::THREADS, C::SMEM, s>>>(c.ntasks, colB, h->row_begin, c.d_task_row, c.d_task_start, c.d_tile_colidx,
                                         (const unsigned char *)c.d_val, (const unsigned char *)d_b, d_c, h->d_error);
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

template <int PREC, int N>
void resources64(TspKernelResources *out)
{
    using C = Cfg64<PREC, N>;
    cudaFuncAttributes attr;
    memset(&attr, 0, sizeof(attr));
    cudaFuncGetAttributes(&attr, k_spmm64<PREC, N>);
    out->threads = C::THREADS;
    out->registers_per_thread = attr.numRegs;
    out->shared_bytes = C::SMEM + (long long)attr.sharedSizeBytes;
    out->tasks_per_block = 1;
    out->iteration_bytes = C::STAGE_BYTES;
}

}  // namespace

int tsp_launch_class64(tsp_handle *h, const void *d_b, float *d_c, int colB, cudaStream_t s)
{
    return h->precision == 0 ? launch64_width<0>(h, d_b, d_c, colB, s) : launch64_width<1>(h, d_b, d_c, colB, s);
}

void tsp_class64_resources(int precision, int colB, TspKernelResources *out)
{
    const int n = tsp_stripe_width(0, colB);
#define TSP_R64(P)                                   \
    do {                                             \
        if (n == 32) resources64<P, 32>(out);        \
        else if (n == 64) resources64<P, 64>(out);   \
        else if (n == 128) resources64<P, 128>(out); \
        else resources64<P, 256>(out);               \
    } while (0)
    if (precision == 0) TSP_R64(0); else TSP_R64(1);
#undef TSP_R64
}
