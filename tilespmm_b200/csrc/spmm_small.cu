// SpMM kernels for the 16-row and 8-row tile classes: warp-level mma.sync with a multi-stage cp.async ring.
//
// They replace upstream stir_spmm_cuda_kernel_v16*/v8* (src/tilespmm_cuda.h:12-1023) and the launch switches
// (src/tilespmm_cuda.h:1634-1708).  Differences that matter on B200:
//   * one warp owns one (task, column stripe) and keeps a 2- to 6-deep ring of gathered B rows in flight
//     (upstream: depth 1 for 16-row tiles, none for 8-row tiles) at 16-24 resident warps per SM;
//   * a stripe is up to 128 columns wide (upstream: 64), so the A tile and the column indices are read
//     once per 128 columns and a gathered row segment is up to 512 contiguous bytes;
//   * every global access is a 16-byte cp.async (B rows, A tile) or a full 32-byte sector store (C);
//   * shared-memory rows are XOR-swizzled in 16-byte chunks so that ldmatrix reads are conflict-free.
// Tile values are consumed in the upstream fragment order (src/csr2tile.h:255-307): one 16-byte (16-row) or
// 8-byte (8-row) load per lane is the MMA operand.
#include "tsp_internal.cuh"

namespace
{

constexpr int WARPS = 4;
// Ring depth per warp.  Occupancy beats depth on B200: on the stencil 24 resident warps with 2 stages outrun 12 warps
// with 4 (0.130 vs 0.165 ms), on R-MAT (64-column stripes, FP16) 2 stages at 8 CTAs per SM outrun 4 stages at 6
// (0.347 vs 0.402 ms).  So: 2 stages for 128- and 64-column stripes, 3 for 32-column ones.
constexpr int ring_stages(int stage_bytes) { return 4608 / stage_bytes < 2 ? 2 : 4608 / stage_bytes; }

__device__ __forceinline__ void cp_async16(void *smem, const void *gmem)
{
    unsigned s = (unsigned)__cvta_generic_to_shared(smem);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(s), "l"(gmem));
}
__device__ __forceinline__ void cp_async16s(unsigned smem, const void *gmem)
{
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(smem), "l"(gmem));
}
// The same copy with an L2 eviction policy.  B is re-read many times per product and by every later product, while a
// tile of A and a row of C pass through once per product: with B about the size of the L2, letting the one-pass data
// go first keeps most of B resident (policies made once per thread with createpolicy).
__device__ __forceinline__ void cp_async16_hint(unsigned smem, const void *gmem, unsigned long long policy)
{
    asm volatile("cp.async.cg.shared.global.L2::cache_hint [%0], [%1], 16, %2;\n" ::"r"(smem), "l"(gmem), "l"(policy));
}
__device__ __forceinline__ unsigned long long policy_evict_first()
{
    unsigned long long p;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;\n" : "=l"(p));
    return p;
}
__device__ __forceinline__ unsigned long long policy_evict_last()
{
    unsigned long long p;
    asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;\n" : "=l"(p));
    return p;
}
__device__ __forceinline__ void store_streaming(float4 *p, float4 v) { __stcs(p, v); }
__device__ __forceinline__ void store_streaming(float2 *p, float2 v) { __stcs(p, v); }
__device__ __forceinline__ void store_streaming(float *p, float v) { __stcs(p, v); }
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }

__device__ __forceinline__ void ldmatrix_x4_trans(unsigned &r0, unsigned &r1, unsigned &r2, unsigned &r3, const void *smem)
{
    unsigned s = (unsigned)__cvta_generic_to_shared(smem);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(s));
}
__device__ __forceinline__ void mma_f16(float *d, unsigned a0, unsigned a1, unsigned a2, unsigned a3, unsigned b0, unsigned b1)
{
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void mma_tf32(float *d, unsigned a0, unsigned a1, unsigned a2, unsigned a3, unsigned b0, unsigned b1)
{
    asm volatile("mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// K = 4 form, used by the 8-row kernel: its A operand is two registers that belong to ONE K column, so a lane feeds two
// MMAs from one 16-byte shared-memory load.
__device__ __forceinline__ void mma_tf32_k4(float *d, unsigned a0, unsigned a1, unsigned b0)
{
    asm volatile("mma.sync.aligned.m16n8k4.row.col.f32.tf32.tf32.f32 {%0,%1,%2,%3}, {%4,%5}, {%6}, {%0,%1,%2,%3};\n"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3]) : "r"(a0), "r"(a1), "r"(b0));
}


#ifndef TSP_SMALL_BULK
#define TSP_SMALL_BULK 0
#endif
// Resident CTAs per SM each instance is compiled for (the register budget of its launch bounds).  The 16-row kernels
// keep 64 accumulator registers per lane at 128 columns: compiled for 5 or 6 CTAs they spill and measure 16 % / 90 %
// slower on the 27-point stencil (TF32), and a third ring slot at 4 CTAs is 4 % slower than two -- the kernel is bound
// by the shared-memory data path (72 % busy) and by issue latency at 16 warps per SM, not by bytes in flight.
constexpr int small_ctas(int cls, int ns) { return cls == 2 ? (ns <= 64 ? 8 : 6) : 4; }
// BULK: the gathered rows and the A tile are fetched by the bulk-copy engine (cp.async.bulk, one copy per row
// segment, completion on an mbarrier per ring slot) instead of per-lane 16-byte cp.async through the load/store
// path; rows then sit unswizzled in shared memory with a 16-byte pad per row to keep the operand loads conflict-free.
// Measured on B200 it is not faster for 512-byte row segments (27-point stencil, TF32, 128 columns: 0.131 ms vs
// 0.129 ms) and much slower for 128-byte segments (R-MAT scale 20, FP16, 64 columns: 0.72 ms vs 0.45 ms), so it is
// compiled out by default (-DTSP_SMALL_BULK=1 enables it).
constexpr bool BULK = TSP_SMALL_BULK != 0;
constexpr unsigned SMALL_WAIT_LIMIT = 1u << 22;

__device__ __forceinline__ void mbar_init_s(unsigned bar, unsigned count) { asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(bar), "r"(count)); }
__device__ __forceinline__ void mbar_expect_tx(unsigned bar, unsigned bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void bulk_g2s(unsigned dst, const void *src, unsigned bytes, unsigned bar)
{
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_wait_s(unsigned bar, unsigned parity)
{
    for (unsigned it = 0; it < SMALL_WAIT_LIMIT; it++)
    {
        unsigned done;
        asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}\n"
                     : "=r"(done) : "r"(bar), "r"(parity) : "memory");
        if (done) return true;
    }
    return false;
}

template <int PREC, int CLS, int NS>
struct SmallCfg
{
    static constexpr int SZ = PREC == 0 ? 2 : 4;
    static constexpr int BM = CLS == 1 ? 16 : 8;
    static constexpr int BN = PREC == 0 ? 16 : 8;
    static constexpr int RB = NS * SZ;                 // bytes of one gathered row segment
    static constexpr int CPR = RB / 16;                // 16-byte chunks per row
    static constexpr int A_BYTES = BM * BN * SZ;       // 512 (16-row) or 256 (8-row)
    static constexpr int RBS = BULK ? RB + 16 : RB;    // row stride in shared memory
    static constexpr int B_BYTES = BN * RBS;
    static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
    static constexpr int STAGES = ring_stages(STAGE_BYTES);
    static constexpr int WARP_BYTES = STAGES * STAGE_BYTES + (BULK ? 64 : 0);   // + one mbarrier per slot
    static constexpr int SMEM = WARPS * WARP_BYTES;
};

// chunk position of 16-byte chunk c of row k inside its shared-memory row
template <int RB>
__device__ __forceinline__ int swz(int c, int k)
{
    if (RB >= 128) return c ^ (k & 7);
    return c ^ ((k >> 1) & 3);
}

// COOP: the four warps of a CTA share ONE (task, stripe): warp w takes tiles w, w+4, ... and the partial blocks are
// added up through shared memory.  Used for launches that would not fill the GPU with one warp per unit: the chain of
// dependent tile fetches of a panel is four times shorter.
template <int PREC, int CLS, int NS, bool COOP>
__global__ void __launch_bounds__(WARPS * 32, small_ctas(CLS, NS))
k_spmm_small(int ntasks, int nstripes, int ldb /* elements */, int row_begin, const uint4 *__restrict__ task_pack,
             const int *__restrict__ tile_colidx, const unsigned char *__restrict__ tile_val,
             const unsigned char *__restrict__ dB, float *__restrict__ dC, int *__restrict__ err, const TspBounds bounds)
{
    using Cfg = SmallCfg<PREC, CLS, NS>;
    constexpr int SZ = Cfg::SZ, BM = Cfg::BM, BN = Cfg::BN, RB = Cfg::RB, CPR = Cfg::CPR, STAGES = Cfg::STAGES, RBS = Cfg::RBS;
    extern __shared__ __align__(128) unsigned char smem_raw[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long unit = COOP ? (long long)blockIdx.x : (long long)blockIdx.x * WARPS + warp;
    if (unit >= (long long)ntasks * nstripes) return;   // COOP: never (one CTA per unit)
    const int task = (int)(unit / nstripes), stripe = (int)(unit - (long long)task * nstripes);
    unsigned char *ring = smem_raw + warp * Cfg::WARP_BYTES;

    const uint4 tp = __ldg(task_pack + task);   // {row word, first tile, end tile, -}: one load per task
    const unsigned int trow = tp.x;
    const bool split = (trow >> 31) != 0;
    const int first_row = (int)(trow & 0x7fffffffu) - row_begin;
    // tiles of this warp: t0, t0 + TS, ... (TS = 1: all tiles of the task)
    constexpr int TS = COOP ? WARPS : 1;
    const int t0 = (int)tp.y + (COOP ? warp : 0);
    int nt = (int)tp.z > t0 ? ((int)tp.z - t0 + TS - 1) / TS : 0;
    bool checked_skip = false;
    if (TSP_CHECKED)
    {
        // checked build: the task must lie inside the class's tiles and its rows inside the caller's C; a task that
        // does not is reported and multiplies nothing (it still takes part in the block's barriers)
        const bool bad_task = (int)tp.y < 0 || (int)tp.z < (int)tp.y || (int)tp.z > bounds.tilenum, bad_rows = first_row < 0 || first_row + BM > bounds.c_rows;
        if (bad_task || bad_rows)
        {
            if (lane == 0) atomicExch(err, bad_task ? 0x21 : 0x22);
            nt = 0;
            checked_skip = true;   // nothing of this task is stored either
        }
    }
    const size_t stripe_bytes = (size_t)stripe * NS * SZ;
    const size_t ldb_bytes = (size_t)ldb * SZ;

    constexpr int NACC = CLS == 1 ? NS / 8 : NS / 16;
    float acc[NACC][4];
#pragma unroll
    for (int i = 0; i < NACC; i++) { acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.0f; }

    // Per-lane constants of the gather.  Chunk q = it*32 + lane of a tile is 16-byte chunk c = lane % CPR of row
    // k = it*KPI + lane/CPR (32 % CPR == 0), so the source column offset and the swizzled destination offset of
    // every copy are loop invariants: one shuffle, one 32x32->64 multiply-add and the copy per 16 bytes.
    static_assert(32 % CPR == 0 || CPR % 32 == 0, "chunks per row must divide or be a multiple of the warp size");
    constexpr int KPI = CPR <= 32 ? 32 / CPR : 1;          // tile rows covered by one warp-wide copy
    constexpr int ITERS = BN * CPR / 32;
    const int c_mine = lane % CPR, k_mine = lane / CPR;
    const unsigned char *gsrc = dB + stripe_bytes + (size_t)c_mine * 16;
    const unsigned ldb_b = (unsigned)ldb_bytes;
    const unsigned ring_s = (unsigned)__cvta_generic_to_shared(ring);
    const unsigned char *a_src = tile_val + (size_t)t0 * Cfg::A_BYTES + lane * 16;
    const int *idx_ptr = tile_colidx + (size_t)t0 * BN + lane;
    // column index of tile row `lane` for the tile that will be issued next
    int idx_next = (nt > 0 && lane < BN) ? __ldg(idx_ptr) : 0;
    if (TSP_CHECKED && (unsigned)idx_next >= (unsigned)bounds.colA) { atomicExch(err, 0x20); idx_next = 0; }

    const unsigned bars = ring_s + STAGES * Cfg::STAGE_BYTES;
    if (BULK)
    {
        if (lane == 0)
        {
            for (int q = 0; q < STAGES; q++) mbar_init_s(bars + 8 * q, 1);
            asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
        }
        __syncwarp();
    }
    const unsigned char *a_tile = tile_val + (size_t)t0 * Cfg::A_BYTES;
    const unsigned char *grow = dB + stripe_bytes;

    const unsigned long long pol_once = policy_evict_first(), pol_keep = policy_evict_last();
    auto issue = [&](int i) {
        const unsigned st = ring_s + (unsigned)(i % STAGES) * Cfg::STAGE_BYTES;
        if (BULK)
        {
            // lane k < BN fetches gathered row k (RB contiguous bytes of B), lane BN the A tile; lane 0 arms the slot
            const unsigned bar = bars + 8 * (i % STAGES);
            if (lane == 0) mbar_expect_tx(bar, Cfg::A_BYTES + BN * RB);
            if (lane < BN) bulk_g2s(st + Cfg::A_BYTES + lane * RBS, grow + (unsigned long long)(unsigned)idx_next * ldb_b, RB, bar);
            else if (lane == BN) bulk_g2s(st, a_tile, Cfg::A_BYTES, bar);
            a_tile += TS * Cfg::A_BYTES;
        }
        else
        {
            if (lane * 16 < Cfg::A_BYTES) cp_async16_hint(st + lane * 16, a_src, pol_once);
            a_src += TS * Cfg::A_BYTES;
            const int idx_mine = idx_next;
#pragma unroll
            for (int it = 0; it < ITERS; it++)
            {
                const int k = it * KPI + k_mine;
                const int col = __shfl_sync(0xffffffffu, idx_mine, k);
                cp_async16_hint(st + Cfg::A_BYTES + k * RB + (swz<RB>(c_mine, k) << 4), gsrc + (unsigned long long)(unsigned)col * ldb_b, pol_keep);
            }
        }
        idx_ptr += TS * BN;
        if (i + 1 < nt && lane < BN) idx_next = __ldg(idx_ptr);
        if (TSP_CHECKED && (unsigned)idx_next >= (unsigned)bounds.colA) { atomicExch(err, 0x20); idx_next = 0; }
    };
    // byte offset of 16-byte chunk `chunk` of gathered row k inside the B part of a slot
    auto boff = [&](int k, int chunk) -> int { return BULK ? k * RBS + chunk * 16 : k * RB + swz<RB>(chunk, k) * 16; };

    bool ok = true;
    for (int i = 0; i < STAGES - 1; i++)
    {
        if (i < nt) issue(i);
        if (!BULK) cp_async_commit();
    }
    for (int i = 0; i < nt; i++)
    {
        if (i + STAGES - 1 < nt) issue(i + STAGES - 1);
        if (BULK)
        {
            ok = __all_sync(0xffffffffu, mbar_wait_s(bars + 8 * (i % STAGES), (i / STAGES) & 1));
            if (!ok)
            {
                // give the copies still in flight one more bounded chance to land, report, and stop
                if (lane == 0) atomicExch(err, 2);
                for (int q = i; q < nt && q < i + STAGES; q++) mbar_wait_s(bars + 8 * (q % STAGES), (q / STAGES) & 1);
                break;
            }
        }
        else
        {
            cp_async_commit();
            cp_async_wait<STAGES - 1>();
            __syncwarp();
        }
        const unsigned char *st = ring + (i % STAGES) * Cfg::STAGE_BYTES;
        const unsigned char *sb = st + Cfg::A_BYTES;
        if constexpr (CLS == 1 && PREC == 0)
        {
            const uint4 a = *reinterpret_cast<const uint4 *>(st + lane * 16);
            const int k = ((lane >> 3) & 1) * 8 + (lane & 7);
#pragma unroll
            for (int nb = 0; nb < NS / 8; nb += 2)
            {
                const int chunk = nb + (lane >> 4);
                unsigned r0, r1, r2, r3;
                ldmatrix_x4_trans(r0, r1, r2, r3, sb + boff(k, chunk));
                mma_f16(acc[nb], a.x, a.y, a.z, a.w, r0, r1);
                mma_f16(acc[nb + 1], a.x, a.y, a.z, a.w, r2, r3);
            }
        }
        else if constexpr (CLS == 1 && PREC == 1)
        {
            // TF32 has no ldmatrix path, so the output columns of the MMAs are permuted instead: lane group
            // g = lane/4 owns the W = NS/8 consecutive columns g*W.., and n-block nb uses column g*W + nb of
            // every group.  A lane then reads its B operands with 16-byte loads (W/4 per K row).
            const uint4 a = *reinterpret_cast<const uint4 *>(st + lane * 16);
            constexpr int W = NS / 8;
            const int k = lane & 3, g = lane >> 2;
            // one K = 8 MMA per n-block: tile rows 0-3 (x) and 4-7 (y) of the lane's column group (5% faster on B200
            // than two K = 4 MMAs here; the 8-row form below measures the same either way)
#pragma unroll
            for (int j = 0; j < W / 4; j++)
            {
                const int chunk = g * (W / 4) + j;
                const uint4 x = *reinterpret_cast<const uint4 *>(sb + boff(k, chunk));
                const uint4 y = *reinterpret_cast<const uint4 *>(sb + boff(k + 4, chunk));
                mma_tf32(acc[4 * j], a.x, a.y, a.z, a.w, x.x, y.x); mma_tf32(acc[4 * j + 1], a.x, a.y, a.z, a.w, x.y, y.y);
                mma_tf32(acc[4 * j + 2], a.x, a.y, a.z, a.w, x.z, y.z); mma_tf32(acc[4 * j + 3], a.x, a.y, a.z, a.w, x.w, y.w);
            }
        }
        else if constexpr (CLS == 2 && PREC == 0)
        {
            const uint2 b = *reinterpret_cast<const uint2 *>(st + lane * 8);
            const int k = (lane >> 4) * 8 + (lane & 7);
#pragma unroll
            for (int mb = 0; mb < NS / 16; mb++)
            {
                const int chunk = mb * 2 + ((lane >> 3) & 1);
                unsigned a0, a1, a2, a3;
                ldmatrix_x4_trans(a0, a1, a2, a3, sb + boff(k, chunk));
                mma_f16(acc[mb], a0, a1, a2, a3, b.x, b.y);
            }
        }
        else
        {
            // same column permutation as the 16-row TF32 kernel: lane group g owns columns g*W .. g*W+W-1 and
            // MMA mb takes column g*W + 2*mb for its row m = g and g*W + 2*mb + 1 for its row m + 8
            const uint2 b = *reinterpret_cast<const uint2 *>(st + lane * 8);
            constexpr int W = NS / 8;
            const int k = lane & 3, g = lane >> 2;
            // two K = 4 MMAs per 16 columns: tile rows 0-3 with b.x, rows 4-7 with b.y; one 16-byte load of a
            // gathered row yields the A operands (columns 2*mb, 2*mb+1 of the lane's group) of two MMAs
#pragma unroll
            for (int j = 0; j < W / 4; j++)
            {
                const int chunk = g * (W / 4) + j;
                const uint4 x = *reinterpret_cast<const uint4 *>(sb + boff(k, chunk));
                const uint4 y = *reinterpret_cast<const uint4 *>(sb + boff(k + 4, chunk));
                mma_tf32_k4(acc[2 * j], x.x, x.y, b.x); mma_tf32_k4(acc[2 * j + 1], x.z, x.w, b.x);
                mma_tf32_k4(acc[2 * j], y.x, y.y, b.y); mma_tf32_k4(acc[2 * j + 1], y.z, y.w, b.y);
            }
        }
        __syncwarp();
    }

    if (!ok) return;
    if constexpr (COOP)
    {
        // warps 1-3 hand their partial block to warp 0 through the (now idle) rings, lane-major
        static_assert(!BULK, "the cooperative form reuses the rings, which hold mbarriers in the bulk-copy variant");
        static_assert((WARPS - 1) * 32 * NACC * 16 <= Cfg::SMEM, "partial blocks must fit the rings");
        float4 *red = reinterpret_cast<float4 *>(smem_raw);
        __syncthreads();   // every warp is done reading its ring
        if (warp > 0)
        {
#pragma unroll
            for (int i = 0; i < NACC; i++) red[((warp - 1) * NACC + i) * 32 + lane] = make_float4(acc[i][0], acc[i][1], acc[i][2], acc[i][3]);
        }
        __syncthreads();
        if (warp > 0) return;
#pragma unroll
        for (int w = 0; w < WARPS - 1; w++)
#pragma unroll
            for (int i = 0; i < NACC; i++)
            {
                const float4 v = red[(w * NACC + i) * 32 + lane];
                acc[i][0] += v.x; acc[i][1] += v.y; acc[i][2] += v.z; acc[i][3] += v.w;
            }
    }
    if (TSP_CHECKED && checked_skip) return;
    // epilogue.  ldc == ldb (upstream uses the padded width as the row stride of both, src/main.cu:173)
    const size_t ldc = (size_t)ldb;
    float *cbase = dC + (size_t)first_row * ldc + (size_t)stripe * NS;
    if constexpr (CLS == 1 && PREC == 1)
    {
        // permuted columns: accumulator (row, n') of n-block nb is C[row][n'*W + nb], n' = (lane%4)*2 + {0,1}
        constexpr int W = NS / 8;
        const int r = lane >> 2;
#pragma unroll
        for (int half = 0; half < 2; half++)
#pragma unroll
            for (int j = 0; j < 2; j++)
            {
                float *p = cbase + (size_t)(r + 8 * half) * ldc + ((lane & 3) * 2 + j) * W;
#pragma unroll
                for (int q = 0; q < W; q += 4)
                {
                    const float v0 = acc[q][half * 2 + j], v1 = acc[q + 1][half * 2 + j], v2 = acc[q + 2][half * 2 + j], v3 = acc[q + 3][half * 2 + j];
                    if (split) { atomicAdd(p + q, v0); atomicAdd(p + q + 1, v1); atomicAdd(p + q + 2, v2); atomicAdd(p + q + 3, v3); }
                    else store_streaming(reinterpret_cast<float4 *>(p + q), make_float4(v0, v1, v2, v3));
                }
            }
    }
    else if constexpr (CLS == 1)
    {
        const int r = lane >> 2, c = (lane & 3) * 2;
#pragma unroll
        for (int nb = 0; nb < NS / 8; nb++)
        {
            float *p0 = cbase + (size_t)r * ldc + nb * 8 + c, *p1 = p0 + 8 * ldc;
            if (split)
            {
                atomicAdd(p0, acc[nb][0]); atomicAdd(p0 + 1, acc[nb][1]);
                atomicAdd(p1, acc[nb][2]); atomicAdd(p1 + 1, acc[nb][3]);
            }
            else
            {
                store_streaming(reinterpret_cast<float2 *>(p0), make_float2(acc[nb][0], acc[nb][1]));
                store_streaming(reinterpret_cast<float2 *>(p1), make_float2(acc[nb][2], acc[nb][3]));
            }
        }
    }
    else if constexpr (PREC == 1)
    {
        // transposed block with permuted columns: accumulator (m, n) of MMA mb is C[row n][g*W + 2*mb + (m >= 8)]
        constexpr int W = NS / 8;
        const int g = lane >> 2, n = (lane & 3) * 2;
#pragma unroll
        for (int j = 0; j < 2; j++)
        {
            float *p = cbase + (size_t)(n + j) * ldc + g * W;
#pragma unroll
            for (int q = 0; q < W / 2; q += 2)
            {
                const float v0 = acc[q][j], v1 = acc[q][2 + j], v2 = acc[q + 1][j], v3 = acc[q + 1][2 + j];
                if (split) { atomicAdd(p + 2 * q, v0); atomicAdd(p + 2 * q + 1, v1); atomicAdd(p + 2 * q + 2, v2); atomicAdd(p + 2 * q + 3, v3); }
                else store_streaming(reinterpret_cast<float4 *>(p + 2 * q), make_float4(v0, v1, v2, v3));
            }
        }
    }
    else
    {
        // the MMA computed the transposed block: accumulator (m, n) is C[row n][column m]
        const int m = lane >> 2, n = (lane & 3) * 2;
#pragma unroll
        for (int mb = 0; mb < NS / 16; mb++)
        {
            float *p = cbase + (size_t)n * ldc + mb * 16 + m;
            if (split)
            {
                atomicAdd(p, acc[mb][0]); atomicAdd(p + ldc, acc[mb][1]);
                atomicAdd(p + 8, acc[mb][2]); atomicAdd(p + ldc + 8, acc[mb][3]);
            }
            else
            {
                store_streaming(p, acc[mb][0]); store_streaming(p + ldc, acc[mb][1]);
                store_streaming(p + 8, acc[mb][2]); store_streaming(p + ldc + 8, acc[mb][3]);
            }
        }
    }
}

template <int PREC, int CLS, int NS>
int launch_one(tsp_handle *h, const void *d_b, float *d_c, int colB, cudaStream_t s)
{
    using Cfg = SmallCfg<PREC, CLS, NS>;
    TspClass &c = h->cls[CLS];
    static bool configured[8] = {false};
    auto kern = k_spmm_small<PREC, CLS, NS, false>;
    auto kern_coop = k_spmm_small<PREC, CLS, NS, true>;
    if (!configured[h->device & 7])
    {
        TSP_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM));
        TSP_CUDA(cudaFuncSetAttribute(kern_coop, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM));
        configured[h->device & 7] = true;
    }
    const int nstripes = colB / NS;
    const long long units = (long long)c.ntasks * nstripes;
    if (units == 0) return TSP_OK;
    TspRange range(CLS == 1 ? "tsp 16-row class kernel" : "tsp 8-row class kernel");
    // One warp per unit fills the GPU only when there are several units per resident warp slot; below that (small
    // matrices) a CTA per unit with the tiles dealt out to its four warps is faster.  Tasks of one or two tiles gain nothing.
    const long long warp_slots = (long long)h->prop.multiProcessorCount * small_ctas(CLS, NS) * WARPS;
    const bool coop = units * WARPS <= warp_slots && (long long)c.tilenum >= 3 * (long long)c.ntasks;
    const int grid = coop ? (int)units : (int)((units + WARPS - 1) / WARPS);
    (coop ? kern_coop : kern)<<<grid, WARPS * 32, Cfg::SMEM, s>>>(c.ntasks, nstripes, colB, h->row_begin, c.d_task_pack, c.d_tile_colidx,
                                            (const unsigned char *)c.d_val, (const unsigned char *)d_b, d_c, h->d_error, tsp_bounds(h, CLS));
    TSP_CUDA(cudaGetLastError());
    h->launches++;
    return TSP_OK;
}

template <int PREC, int CLS>
int launch_width(tsp_handle *h, const void *d_b, float *d_c, int colB, cudaStream_t s)
{
    switch (tsp_stripe_width(CLS, colB))
    {
    case 32: return launch_one<PREC, CLS, 32>(h, d_b, d_c, colB, s);
    case 128: return launch_one<PREC, CLS, 128>(h, d_b, d_c, colB, s);
    default: return launch_one<PREC, CLS, 64>(h, d_b, d_c, colB, s);
    }
}

template <int PREC, int CLS, int NS>
void resources_one(TspKernelResources *out)
{
    using Cfg = SmallCfg<PREC, CLS, NS>;
    cudaFuncAttributes attr;
    memset(&attr, 0, sizeof(attr));
    cudaFuncGetAttributes(&attr, k_spmm_small<PREC, CLS, NS, false>);
    out->threads = WARPS * 32;
    out->registers_per_thread = attr.numRegs;
    out->shared_bytes = Cfg::SMEM + (long long)attr.sharedSizeBytes;
    out->tasks_per_block = WARPS;
    out->iteration_bytes = WARPS * Cfg::STAGE_BYTES;
}

}  // namespace

// Zeroes the C rows of split panels (their tasks accumulate with atomics).  Upstream clears all of C
// with cudaMemset outside its timers (src/csr2tile.h:1024, 1038).
__global__ void k_clear_split_rows(int nsplit, const int *__restrict__ split_row, int bm, int row_begin, int ldc, float *__restrict__ dC)
{
    const int p = blockIdx.x;
    if (p >= nsplit) return;
    float4 *dst = reinterpret_cast<float4 *>(dC + (size_t)(split_row[p] - row_begin) * ldc);
    const int n4 = bm * ldc / 4;
    for (int i = threadIdx.x; i < n4; i += blockDim.x) dst[i] = make_float4(0.f, 0.f, 0.f, 0.f);
}

int tsp_launch_clear(tsp_handle *h, float *d_c, int colB, cudaStream_t s)
{
    for (int k = 0; k < 3; k++)
    {
        TspClass &c = h->cls[k];
        if (c.tilenum == 0 || c.nsplit == 0) continue;
        k_clear_split_rows<<<c.nsplit, 256, 0, s>>>(c.nsplit, c.d_split_row, c.BM, h->row_begin, colB, d_c);
        TSP_CUDA(cudaGetLastError());
        h->launches++;
    }
    return TSP_OK;
}

int tsp_launch_small(tsp_handle *h, int cls, const void *d_b, float *d_c, int colB, cudaStream_t s)
{
    if (h->precision == 0)
        return cls == 1 ? launch_width<0, 1>(h, d_b, d_c, colB, s) : launch_width<0, 2>(h, d_b, d_c, colB, s);
    return cls == 1 ? launch_width<1, 1>(h, d_b, d_c, colB, s) : launch_width<1, 2>(h, d_b, d_c, colB, s);
}

void tsp_small_resources(int precision, int cls, int colB, TspKernelResources *out)
{
    const int ns = tsp_stripe_width(cls, colB);
#define TSP_RES(P, C)                                                  \
    do {                                                               \
        if (ns == 32) resources_one<P, C, 32>(out);                    \
        else if (ns == 64) resources_one<P, C, 64>(out);               \
        else resources_one<P, C, 128>(out);                            \
    } while (0)
    if (precision == 0) { if (cls == 1) TSP_RES(0, 1); else TSP_RES(0, 2); }
    else { if (cls == 1) TSP_RES(1, 1); else TSP_RES(1, 2); }
#undef TSP_RES
}
