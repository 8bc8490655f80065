// SpMM kernels for the 16-row and 8-row tile classes: warp-level mma.sync with a multi-stage cp.async ring.
//
// They replace upstream stir_spmm_cuda_kernel_v16*/v8* (src/tilespmm_cuda.h:12-1023) and the launch switches
// (src/tilespmm_cuda.h:1634-1708).  Differences that matter on B200:
//   * one warp owns one (task, column stripe) and keeps a 2- or 3-deep ring of gathered B rows in flight
//     (upstream: depth 1 for 16-row tiles, none for 8-row tiles) at 16-32 resident warps per SM;
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

// 16-byte asynchronous copy global -> shared with an L2 eviction policy.  B is re-read many times per product and by every later product, while a
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

// Shared-memory loads by 32-bit shared address: the operand addresses below are built from a per-lane constant, the
// slot base and one XOR per load, all in 32-bit arithmetic.
__device__ __forceinline__ uint4 lds128(unsigned s)
{
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];\n" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(s));
    return v;
}
__device__ __forceinline__ uint2 lds64(unsigned s)
{
    uint2 v;
    asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];\n" : "=r"(v.x), "=r"(v.y) : "r"(s));
    return v;
}
__device__ __forceinline__ void ldmatrix_x4_trans(unsigned &r0, unsigned &r1, unsigned &r2, unsigned &r3, unsigned s)
{
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(s));
}
__device__ __forceinline__ void mma_f16(float *d, unsigned a0, unsigned a1, unsigned a2, unsigned a3, unsigned b0, unsigned b1)
{
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
// K = 8 form of the TF32 MMA: a0/a1 are rows m, m + 8 of K column k, a2/a3 the same rows of K column k + 4.
__device__ __forceinline__ void mma_tf32_k8(float *d, unsigned a0, unsigned a1, unsigned a2, unsigned a3, unsigned b0, unsigned b1)
{
    asm volatile("mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
// K = 4 form of the TF32 MMA: its A operand is two registers that belong to ONE K column, so a lane feeds two MMAs from
// one 16-byte shared-memory load.
__device__ __forceinline__ void mma_tf32_k4(float *d, unsigned a0, unsigned a1, unsigned b0)
{
    asm volatile("mma.sync.aligned.m16n8k4.row.col.f32.tf32.tf32.f32 {%0,%1,%2,%3}, {%4,%5}, {%6}, {%0,%1,%2,%3};\n"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3]) : "r"(a0), "r"(a1), "r"(b0));
}


// Resident CTAs per SM each instance is compiled for (the register budget of its launch bounds).  The 16-row kernels
// keep 64 accumulator registers per lane at 128 columns and spill when compiled for 5 or 6 CTAs.
constexpr int small_ctas(int cls, int ns) { return cls == 2 ? (ns <= 64 ? 8 : 6) : 4; }

template <int PREC, int CLS, int NS>
struct SmallCfg
{
    static constexpr int SZ = PREC == 0 ? 2 : 4;
    static constexpr int BM = CLS == 1 ? 16 : 8;
    static constexpr int BN = PREC == 0 ? 16 : 8;
    static constexpr int RB = NS * SZ;                 // bytes of one gathered row segment
    static constexpr int CPR = RB / 16;                // 16-byte chunks per row
    static constexpr int A_BYTES = BM * BN * SZ;       // 512 (16-row) or 256 (8-row)
    static constexpr int B_BYTES = BN * RB;
    static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
    static constexpr int STAGES = ring_stages(STAGE_BYTES);
    static constexpr int WARP_BYTES = STAGES * STAGE_BYTES;
    static constexpr int SMEM = WARPS * WARP_BYTES;
    // the operand addresses are formed as (slot base + per-lane constant) ^ (small multiple of 16): that equals an XOR on the
    // chunk field of a row (address bits 4-7 at most) alone: slots and the B part inside them start on 256-byte boundaries
    static_assert(A_BYTES % 256 == 0 && STAGE_BYTES % 256 == 0 && WARP_BYTES % 256 == 0 && RB % 64 == 0, "slot layout");
};

// Gathered row k keeps its 16-byte chunk c at chunk position c ^ key(k) of its shared-memory row, so that the operand
// loads (several rows, same chunk) and the copies (one row, all chunks) are both free of bank conflicts.
template <int RB>
__device__ __forceinline__ int swz_key(int k)
{
    return RB >= 128 ? (k & 7) : ((k >> 1) & 3);
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
    constexpr int SZ = Cfg::SZ, BM = Cfg::BM, BN = Cfg::BN, RB = Cfg::RB, CPR = Cfg::CPR, STAGES = Cfg::STAGES;
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long unit = COOP ? (long long)blockIdx.x : (long long)blockIdx.x * WARPS + warp;
    if (unit >= (long long)ntasks * nstripes) return;   // COOP: never (one CTA per unit)
    const int task = (int)(unit / nstripes), stripe = (int)(unit - (long long)task * nstripes);

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
    // k = it*KPI + lane/CPR (32 % CPR == 0).  The destination of copy `it` inside the B part of a slot is
    //   k*RB + ((c ^ key(k)) << 4)  =  (cp_base ^ (key(it*KPI) << 4)) + it*KPI*RB,   cp_base = k0*RB + ((c ^ key(k0)) << 4),
    // with k0 = lane/CPR (key(it*KPI + k0) = key(it*KPI) ^ key(k0): KPI is a power of two above k0), so a copy costs one
    // shuffle, one 32x32->64 multiply-add, one XOR with a constant and the copy itself.
    static_assert(32 % CPR == 0 || CPR % 32 == 0, "chunks per row must divide or be a multiple of the warp size");
    constexpr int KPI = CPR <= 32 ? 32 / CPR : 1;          // tile rows covered by one warp-wide copy
    constexpr int ITERS = BN * CPR / 32;
    static_assert(RB >= 128 || KPI % 2 == 0, "64-byte rows: the swizzle key drops bit 0 of the row");
    const int c_mine = lane % CPR, k_mine = lane / CPR;
    const unsigned char *gsrc = dB + stripe_bytes + (size_t)c_mine * 16;
    const unsigned ldb_b = (unsigned)ldb_bytes;
    const unsigned smem_s = (unsigned)__cvta_generic_to_shared(smem_raw);
    if (smem_s & 255u)   // the XOR addressing below needs the slots on 256-byte boundaries; same outcome for every thread
    {
        if (threadIdx.x == 0) atomicExch(err, 4);
        return;
    }
    const unsigned ring_s = smem_s + (unsigned)warp * Cfg::WARP_BYTES;
    const unsigned cp_base = Cfg::A_BYTES + (unsigned)k_mine * RB + ((unsigned)(c_mine ^ swz_key<RB>(k_mine)) << 4);
    const unsigned char *a_src = tile_val + (size_t)t0 * Cfg::A_BYTES + lane * 16;
    const int *idx_ptr = tile_colidx + (size_t)t0 * BN + lane;
    // column index of tile row `lane` for the tile that will be issued next
    int idx_next = (nt > 0 && lane < BN) ? __ldg(idx_ptr) : 0;
    if (TSP_CHECKED && (unsigned)idx_next >= (unsigned)bounds.colA) { atomicExch(err, 0x20); idx_next = 0; }

    const unsigned long long pol_once = policy_evict_first(), pol_keep = policy_evict_last();
    auto issue = [&](int i) {
        const unsigned st = ring_s + (unsigned)(i % STAGES) * Cfg::STAGE_BYTES;
        if (lane * 16 < Cfg::A_BYTES) cp_async16_hint(st + lane * 16, a_src, pol_once);
        a_src += TS * Cfg::A_BYTES;
        const int idx_mine = idx_next;
        const unsigned dst = st + cp_base;
#pragma unroll
        for (int it = 0; it < ITERS; it++)
        {
            const int col = __shfl_sync(0xffffffffu, idx_mine, it * KPI + k_mine);
            cp_async16_hint((dst ^ ((unsigned)swz_key<RB>(it * KPI) << 4)) + (unsigned)(it * KPI * RB), gsrc + (unsigned long long)(unsigned)col * ldb_b, pol_keep);
        }
        idx_ptr += TS * BN;
        if (i + 1 < nt && lane < BN) idx_next = __ldg(idx_ptr);
        if (TSP_CHECKED && (unsigned)idx_next >= (unsigned)bounds.colA) { atomicExch(err, 0x20); idx_next = 0; }
    };

    // Per-lane constants of the operand loads: a lane reads chunk c0 + n*step (n = 0, 1, ...) of tile row kx (and of row
    // kx + 4 in the TF32 forms), i.e. the bytes at (slot + op_x) ^ (n*step << 4) -- one XOR with a constant per load.
    //   FP16 16-row (ldmatrix.x4.trans): row ((lane>>3)&1)*8 + (lane&7), chunks nb + (lane>>4), nb = 0, 2, ...
    //   FP16 8-row  (ldmatrix.x4.trans): row (lane>>4)*8 + (lane&7),     chunks 2*mb + ((lane>>3)&1)
    //   TF32: lane group g = lane/4 owns the W = NS/8 consecutive output columns g*W.. (W/4 chunks), row lane%4 (+4)
    unsigned op_x, op_y = 0;
    if constexpr (PREC == 0)
    {
        const int kx = CLS == 1 ? ((lane >> 3) & 1) * 8 + (lane & 7) : (lane >> 4) * 8 + (lane & 7);
        const int c0 = CLS == 1 ? (lane >> 4) : ((lane >> 3) & 1);
        op_x = Cfg::A_BYTES + (unsigned)kx * RB + ((unsigned)(c0 ^ swz_key<RB>(kx)) << 4);
    }
    else
    {
        const int kx = lane & 3, c0 = (lane >> 2) * (NS / 32);
        op_x = Cfg::A_BYTES + (unsigned)kx * RB + ((unsigned)(c0 ^ swz_key<RB>(kx)) << 4);
        op_y = Cfg::A_BYTES + (unsigned)(kx + 4) * RB + ((unsigned)(c0 ^ swz_key<RB>(kx + 4)) << 4);
    }

    // The slot of a tile is given back as soon as its last operand is in registers: the MMAs of all but the last step of
    // the tile run from loads issued as they go, then the operands of the last step are loaded, the tile STAGES ahead is
    // requested into the slot, and the last MMAs run while that request is already in flight -- all STAGES slots of a warp
    // are in flight except during the loads of one.  (Deferring more steps costs registers: two steps measure 3 % slower
    // on the 27-point stencil, all four spill and run 1.7x slower.)
    for (int i = 0; i < STAGES; i++)
    {
        if (i < nt) issue(i);
        cp_async_commit();
    }
    for (int i = 0; i < nt; i++)
    {
        cp_async_wait<STAGES - 1>();
        __syncwarp();
        const unsigned st = ring_s + (unsigned)(i % STAGES) * Cfg::STAGE_BYTES;
        auto release = [&]() {
            __syncwarp();   // every lane has its operands: the slot may be overwritten
            if (i + STAGES < nt) issue(i + STAGES);
            cp_async_commit();
        };
        if constexpr (CLS == 1 && PREC == 0)
        {
            constexpr int NP = NS / 16, D = 1;   // pairs of n-blocks; deferred pairs
            const uint4 a = lds128(st + lane * 16);
#pragma unroll
            for (int p = 0; p < NP - D; p++)
            {
                unsigned r0, r1, r2, r3;
                ldmatrix_x4_trans(r0, r1, r2, r3, (st + op_x) ^ (unsigned)(p << 5));
                mma_f16(acc[2 * p], a.x, a.y, a.z, a.w, r0, r1);
                mma_f16(acc[2 * p + 1], a.x, a.y, a.z, a.w, r2, r3);
            }
            unsigned r[D][4];
#pragma unroll
            for (int q = 0; q < D; q++) ldmatrix_x4_trans(r[q][0], r[q][1], r[q][2], r[q][3], (st + op_x) ^ (unsigned)((NP - D + q) << 5));
            release();
#pragma unroll
            for (int q = 0; q < D; q++)
            {
                mma_f16(acc[2 * (NP - D + q)], a.x, a.y, a.z, a.w, r[q][0], r[q][1]);
                mma_f16(acc[2 * (NP - D + q) + 1], a.x, a.y, a.z, a.w, r[q][2], r[q][3]);
            }
        }
        else if constexpr (CLS == 2 && PREC == 0)
        {
            constexpr int MB = NS / 16, D = 1;
            const uint2 b = lds64(st + lane * 8);
#pragma unroll
            for (int mb = 0; mb < MB - D; mb++)
            {
                unsigned a0, a1, a2, a3;
                ldmatrix_x4_trans(a0, a1, a2, a3, (st + op_x) ^ (unsigned)(mb << 5));
                mma_f16(acc[mb], a0, a1, a2, a3, b.x, b.y);
            }
            unsigned r[D][4];
#pragma unroll
            for (int q = 0; q < D; q++) ldmatrix_x4_trans(r[q][0], r[q][1], r[q][2], r[q][3], (st + op_x) ^ (unsigned)((MB - D + q) << 5));
            release();
#pragma unroll
            for (int q = 0; q < D; q++) mma_f16(acc[MB - D + q], r[q][0], r[q][1], r[q][2], r[q][3], b.x, b.y);
        }
        else if constexpr (CLS == 1)
        {
            // TF32 has no ldmatrix path, so the output columns of the MMAs are permuted instead: lane group g = lane/4
            // owns the W = NS/8 consecutive columns g*W.., read with 16-byte loads.  The product is formed transposed
            // (the gathered rows are the m16 x k4 operand, the tile the k4 x n8 operand) once per half of the tile's rows,
            // so that the two registers of an operand are neighbours of ONE load: the 16 x 8 x 8 form needs its two B
            // registers from two different loads and pays two register moves per MMA for it.  The fragment-order tile
            // is exactly the four k4 x n8 operands: a.x rows 0-7 / columns 0-3, a.y rows 8-15 / columns 0-3, a.z and a.w
            // the same rows for columns 4-7.  Accumulators 0 .. W/2-1: rows 0-7, W/2 .. W-1: rows 8-15.
            constexpr int NJ = NS / 32, D = 1, H = NS / 16;
            const uint4 a = lds128(st + lane * 16);
            auto mmas = [&](int j, const uint4 &x, const uint4 &y) {
                mma_tf32_k4(acc[2 * j], x.x, x.y, a.x); mma_tf32_k4(acc[2 * j + 1], x.z, x.w, a.x);
                mma_tf32_k4(acc[H + 2 * j], x.x, x.y, a.y); mma_tf32_k4(acc[H + 2 * j + 1], x.z, x.w, a.y);
                mma_tf32_k4(acc[2 * j], y.x, y.y, a.z); mma_tf32_k4(acc[2 * j + 1], y.z, y.w, a.z);
                mma_tf32_k4(acc[H + 2 * j], y.x, y.y, a.w); mma_tf32_k4(acc[H + 2 * j + 1], y.z, y.w, a.w);
            };
#pragma unroll
            for (int j = 0; j < NJ - D; j++) mmas(j, lds128((st + op_x) ^ (unsigned)(j << 4)), lds128((st + op_y) ^ (unsigned)(j << 4)));
            uint4 xs[D], ys[D];
#pragma unroll
            for (int q = 0; q < D; q++) { xs[q] = lds128((st + op_x) ^ (unsigned)((NJ - D + q) << 4)); ys[q] = lds128((st + op_y) ^ (unsigned)((NJ - D + q) << 4)); }
            release();
#pragma unroll
            for (int q = 0; q < D; q++) mmas(NJ - D + q, xs[q], ys[q]);
        }
        else
        {
            // same column permutation: lane group g owns columns g*W .. g*W+W-1 and MMA mb takes column g*W + 2*mb for
            // its row m = g and g*W + 2*mb + 1 for its row m + 8.  One K = 8 MMA per 16 columns: its A operand is two
            // registers of the load of gathered row k and two of row k + 4 (the compiler moves them into one quad), its B
            // operand the 8-byte tile fragment.  The tensor pipe takes as long for a K = 4 MMA as for a K = 8 one, so this
            // halves its load: the same time in a short burst, 2 % faster under the power cap of a long run than two
            // K = 4 MMAs without the moves
            constexpr int NJ = NS / 32, D = 1;
            const uint2 b = lds64(st + lane * 8);
            auto mmas = [&](int j, const uint4 &x, const uint4 &y) {
                mma_tf32_k8(acc[2 * j], x.x, x.y, y.x, y.y, b.x, b.y); mma_tf32_k8(acc[2 * j + 1], x.z, x.w, y.z, y.w, b.x, b.y);
            };
#pragma unroll
            for (int j = 0; j < NJ - D; j++) mmas(j, lds128((st + op_x) ^ (unsigned)(j << 4)), lds128((st + op_y) ^ (unsigned)(j << 4)));
            uint4 xs[D], ys[D];
#pragma unroll
            for (int q = 0; q < D; q++) { xs[q] = lds128((st + op_x) ^ (unsigned)((NJ - D + q) << 4)); ys[q] = lds128((st + op_y) ^ (unsigned)((NJ - D + q) << 4)); }
            release();
#pragma unroll
            for (int q = 0; q < D; q++) mmas(NJ - D + q, xs[q], ys[q]);
        }
    }

    if constexpr (COOP)
    {
        // warps 1-3 hand their partial block to warp 0 through the (now idle) rings, lane-major
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
    if constexpr (PREC == 1)
    {
        // transposed blocks with permuted columns: accumulator (m, n) of MMA mb of row half h is
        // C[row 8*h + n][g*W + 2*mb + (m >= 8)]
        constexpr int W = NS / 8, HALVES = CLS == 1 ? 2 : 1;
        const int g = lane >> 2, n = (lane & 3) * 2;
#pragma unroll
        for (int h = 0; h < HALVES; h++)
#pragma unroll
            for (int j = 0; j < 2; j++)
            {
                float *p = cbase + (size_t)(8 * h + n + j) * ldc + g * W;
#pragma unroll
                for (int q = 0; q < W / 2; q += 2)
                {
                    const float v0 = acc[h * (W / 2) + q][j], v1 = acc[h * (W / 2) + q][2 + j], v2 = acc[h * (W / 2) + q + 1][j], v3 = acc[h * (W / 2) + q + 1][2 + j];
                    if (split) { atomicAdd(p + 2 * q, v0); atomicAdd(p + 2 * q + 1, v1); atomicAdd(p + 2 * q + 2, v2); atomicAdd(p + 2 * q + 3, v3); }
                    else store_streaming(reinterpret_cast<float4 *>(p + 2 * q), make_float4(v0, v1, v2, v3));
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
