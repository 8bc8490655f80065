// SpMM kernel for the 64-row tile class: tcgen05.mma with the accumulator in tensor memory (sm_100a), fed from
// PACKED tiles.
//
// Replaces upstream stir_spmm_cuda_kernel_v64* (src/tilespmm_cuda.h:1025-1632) and switch_tilespmm_cuda_v64
// (src/tilespmm_cuda.h:1710-1744).  Upstream keeps every 64-row tile as a dense, zero-padded 4 KB block
// (src/csr2tile.h:309-373); on a stencil 95% of those bytes are zeros.  Here a tile is a RECORD in one byte array:
//   packed record   for a tile with n <= REC_MAX_VALS entries: n_pad = n rounded up to 8 positions of 16 bits (the
//                   element index of the entry inside the 4 KB operand tile; 0xffff in the padding) followed by n_pad
//                   values, both in row-major order of the entries;
//   dense record    the 4 KB tile in the K-major core-matrix order tcgen05.mma reads -- for fuller tiles.
// rec[t] is the record's offset in 16-byte units, bit 31 set for a dense record.
//
// One CTA owns one task (a 64-row panel or a slice of a split panel) and one column stripe of up to 256 columns, so
// the tile records and column indices are read once per 256 columns (upstream: once per 64).  Roles:
//   warps 0..PW-1   B producers (PW = 8 for stripes of 128 columns and more, else 4).  Together they gather the B rows
//              named by tile_colidx with 16-byte cp.async straight into the swizzled MN-major operand layout of the ring
//              slot, every thread a fixed few chunks of every tile; nobody waits for the data (each thread leaves a
//              cp.async.mbarrier.arrive on the slot's barrier), so every free slot is in flight.  In the
//              TMA form one lane issues cp.async.bulk.tensor ... tile::gather4 requests instead.  What bounds a
//              gather-fed kernel on this GPU is the number of independent warps that issue loads (a warp issues an
//              instruction every ~11 cycles), which is why the rows of ONE tile are spread over all producer threads.
//              Warps 0-3 are also the epilogue: tcgen05.ld of the 64 x N FP32 accumulator -> C.
//   next NE warps  expanders.  Expander e owns tiles e, e+NE, ...: it copies the tile's record into a private buffer one
//              tile ahead (cp.async) and expands it into the slot's 4 KB A area in operand order -- zero fill plus one
//              store per value; for a dense record one 4 KB bulk copy -- then arrives on the slot's barrier.
//   last warp  allocates tensor memory; one lane issues two tcgen05.mma (M=64, N=stripe, K=16 FP16 / K=8 TF32) per
//              tile and releases ring slots with tcgen05.commit.
// The accumulator of a whole task stays in tensor memory (64 lanes x N columns) and is written once, with vector
// stores, or vector red.global.add for the slices of a split panel.
// Every wait on an mbarrier is bounded; when one runs out the kernel records it in *err, frees its tensor memory and
// returns.
#include <cuda.h>

#include "tsp_internal.cuh"

namespace
{

constexpr unsigned WAIT_LIMIT = 1u << 20;
constexpr unsigned WAIT_PARK_NS = 2000;
#ifndef TSP64_NE
#define TSP64_NE 2                     // expander warps
#endif

template <int PREC, int N>
struct Cfg64
{
    static constexpr int SZ = PREC == 0 ? 2 : 4;
    static constexpr int BNK = PREC == 0 ? 32 : 16;           // K extent of a tile = gathered rows per tile
    static constexpr int A_BYTES = 64 * BNK * SZ;             // 4096
    static constexpr int RB = N * SZ;                         // bytes of one gathered row segment
    static constexpr int CPR = RB / 16;                       // 16-byte chunks per row segment
    static constexpr int B_BYTES = BNK * RB;
    static constexpr int PW = N >= 128 ? 8 : 4;               // B producer warps
    static constexpr int NE = TSP64_NE;                       // expander warps
    static constexpr int THREADS = (PW + NE + 1) * 32;
    static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
    static constexpr int B_ITERS = (BNK * CPR) / (PW * 32);   // copies per producer thread per tile
    static constexpr int KPI = PW * 32 / CPR;                 // tile rows covered by one CTA-wide copy
    // ring depth: a slot is reused STAGES tiles later and all STAGES slots can be in flight to memory
#ifdef TSP64_STAGES
    static constexpr int STAGES = TSP64_STAGES;
#else
    static constexpr int STAGES = N >= 128 ? 4 : (N == 64 ? 6 : 8);
#endif
    static_assert(B_ITERS >= 1, "unsupported pipeline shape");
    // packed records
    static constexpr int MASK_BYTES = 64 * BNK / 8;           // 128 (TF32) / 256 (FP16)
    static constexpr int REC_MAX_VALS = TSP_REC_MAX_VALS(PREC);
    static constexpr int REC_BYTES = REC_MAX_VALS * (2 + SZ);   // positions + values of the fullest packed record
    static constexpr int REC_CHUNKS = REC_BYTES / 16;
    static constexpr int SMEM = STAGES * STAGE_BYTES + NE * 2 * REC_BYTES + 1024;  // + slack to align the ring to 1 KB
    // Shared-memory layout of the gathered rows (the MN-major B operand):
    //   FP16, rows >= 128 B : 128-byte swizzle, atoms of 8 K-rows x 128 B, 16-byte chunks XORed with the row
    //   FP16, 64-byte rows  : 64-byte swizzle, atoms of 8 K-rows x 64 B
    //   TF32                : the only MN-major mode for 32-bit operands, "128-byte swizzle with 32-byte
    //                         atomicity": atoms of 4 K-rows x 128 B, 32-byte chunks XORed with the row
    static constexpr int MODE = PREC == 1 ? 1 : (RB >= 128 ? 2 : 4);   // layout-type field of the descriptor
    static constexpr int ATOM_ROWS = PREC == 1 ? 4 : 8;
    static constexpr int BOX_BYTES = RB >= 128 ? 128 : 64;    // bytes of one atom row = inner extent of one gather4 box
    static constexpr int BOX_COLS = BOX_BYTES / SZ;
    static constexpr int NBOX = RB / BOX_BYTES;
    static constexpr int ATOM_BYTES = ATOM_ROWS * BOX_BYTES;
    static constexpr int KATOMS = BNK / ATOM_ROWS;            // atoms along K per tile (4)
    static constexpr int KATOMS_PER_MMA = 2;                  // K = 16 halves = 2x8 rows / 8 floats = 2x4 rows
    static constexpr int TMEM_COLS = N < 32 ? 32 : N;
    // tcgen05.alloc blocks until columns are free; it cannot block forever because the CTAs that fit one SM by
    // shared memory never ask for more than the 512 columns together
    static constexpr int MAX_CTAS_BY_SMEM = (227 * 1024) / SMEM;
    static_assert(MAX_CTAS_BY_SMEM >= 1 && MAX_CTAS_BY_SMEM * TMEM_COLS <= 512, "resident CTAs must fit tensor memory");
};

__device__ __forceinline__ unsigned smem_u32(const void *p) { return (unsigned)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void cp_async16(unsigned smem, const void *gmem)
{
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(smem), "l"(gmem));
}
// The same copy with an L2 eviction policy: gathered rows of B are re-read many times per product and by every later
// product, a tile record and a row of C pass through once -- with B about the size of the L2, letting the one-pass data
// go first keeps most of B resident.
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
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int K>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(K) : "memory"); }

__device__ __forceinline__ void mbar_init(unsigned bar, unsigned count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(bar), "r"(count));
}
// arrive on the mbarrier when every cp.async this thread has issued so far has landed; the thread itself does not wait
__device__ __forceinline__ void cp_async_arrive(unsigned bar)
{
    asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];\n" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive(unsigned bar)
{
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(bar) : "memory");
}
// announces bytes that asynchronous copies will deliver to this phase, without arriving
__device__ __forceinline__ void mbar_expect_tx_only(unsigned bar, unsigned bytes)
{
    asm volatile("mbarrier.expect_tx.relaxed.cta.shared::cta.b64 [%0], %1;\n" ::"r"(bar), "r"(bytes) : "memory");
}
// one bulk copy (the copy engine, no per-thread work): global -> shared, completion counted in bytes on the mbarrier
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
// bounded wait: false when the phase did not complete within WAIT_LIMIT polls.  Every poll may park the thread for up to
// WAIT_PARK_NS (the hardware wakes it when the phase completes), so a waiting thread issues few instructions and the
// whole wait is bounded by about WAIT_LIMIT * WAIT_PARK_NS = 2 s.
__device__ __forceinline__ bool mbar_wait(unsigned bar, unsigned parity)
{
    for (unsigned it = 0; it < WAIT_LIMIT; it++)
    {
        unsigned done;
        asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\tselp.u32 %0, 1, 0, p;\n\t}\n"
                     : "=r"(done) : "r"(bar), "r"(parity), "r"(WAIT_PARK_NS) : "memory");
        if (done) return true;
    }
    return false;
}
// the same wait by one lane of a warp, outcome broadcast to all lanes
__device__ __forceinline__ bool mbar_wait_warp(unsigned bar, unsigned parity, int lane)
{
    unsigned ok = 1;
    if (lane == 0) ok = mbar_wait(bar, parity) ? 1u : 0u;
    return __shfl_sync(0xffffffffu, ok, 0) != 0;
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
__device__ __forceinline__ void tmem_ld16(unsigned taddr, unsigned (&r)[16])
{
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 "
                 "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
                   "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
                 : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
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

// Byte offset, inside the B part of a ring slot, of 16-byte chunk c of gathered row k (see the layout table in Cfg64).
template <typename C>
__device__ __forceinline__ unsigned b_chunk_offset(int k, int c)
{
    if (C::MODE == 2) { const int ka = k >> 3, kr = k & 7; return ((c >> 3) * C::KATOMS + ka) * 1024 + kr * 128 + (((c & 7) ^ kr) << 4); }
    if (C::MODE == 4) { const int ka = k >> 3, kr = k & 7; return ka * 512 + kr * 64 + ((c ^ ((kr >> 1) & 3)) << 4); }
    const int ka = k >> 2, kr = k & 3;
    return ((c >> 3) * C::KATOMS + ka) * 512 + kr * 128 + (((((c & 7) >> 1) ^ kr) << 5) | ((c & 1) << 4));
}

// Expands the packed record at shared address `rec` (n_pad 16-bit positions, then n_pad values) into the 4 KB A area at
// shared address `a` (K-major core matrices, tsp_umma_index): zero fill, then one store per value.  A position is the
// element index inside the operand tile, so a lane's work per value is two loads and one store; 0xffff marks padding.
template <int PREC>
__device__ __forceinline__ void expand_record(unsigned rec, unsigned n_pad, unsigned a, int lane)
{
    constexpr int SZ = PREC == 0 ? 2 : 4;
    __syncwarp();   // the record was copied in by all lanes of the warp
#pragma unroll
    for (int q = 0; q < 8; q++)
        asm volatile("st.shared.v4.b32 [%0], {%1,%1,%1,%1};\n" ::"r"(a + (unsigned)(q * 32 + lane) * 16), "r"(0u) : "memory");
    __syncwarp();   // the zero fill of every lane is ordered before any lane's value stores
    const unsigned vals = rec + n_pad * 2;
    for (unsigned j = lane; j < n_pad; j += 32)
    {
        unsigned short u;
        asm volatile("ld.shared.u16 %0, [%1];\n" : "=h"(u) : "r"(rec + j * 2));
        if (u == 0xffffu) continue;
        if constexpr (PREC == 1)
        {
            unsigned v;
            asm volatile("ld.shared.b32 %0, [%1];\n" : "=r"(v) : "r"(vals + j * 4));
            asm volatile("st.shared.b32 [%0], %1;\n" ::"r"(a + (unsigned)u * 4), "r"(v) : "memory");
        }
        else
        {
            unsigned short v;
            asm volatile("ld.shared.b16 %0, [%1];\n" : "=h"(v) : "r"(vals + j * 2));
            asm volatile("st.shared.b16 [%0], %1;\n" ::"r"(a + (unsigned)u * 2), "h"(v) : "memory");
        }
    }
}

template <int PREC, int N, bool TMA>
__global__ void __launch_bounds__(Cfg64<PREC, N>::THREADS, (Cfg64<PREC, N>::MAX_CTAS_BY_SMEM > 4 ? 4 : Cfg64<PREC, N>::MAX_CTAS_BY_SMEM))
k_spmm64(const __grid_constant__ CUtensorMap bmap, int ntasks, int ldb, int row_begin, const unsigned int *__restrict__ task_row,
         const int *__restrict__ task_start, const int *__restrict__ tile_colidx, const unsigned int *__restrict__ rec_ptr,
         const unsigned char *__restrict__ pack, const unsigned char *__restrict__ dB, float *__restrict__ dC, int *__restrict__ err,
         const TspBounds bounds)
{
    using C = Cfg64<PREC, N>;
    constexpr int S = C::STAGES, PW = C::PW, NE = C::NE;
    extern __shared__ unsigned char smem_raw[];
    __shared__ __align__(8) unsigned long long bars[2 * C::STAGES + 1];
    __shared__ unsigned tmem_slot;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, tid = threadIdx.x;
    const int task = blockIdx.x, stripe = blockIdx.y;
    const unsigned ring = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const unsigned recs = ring + S * C::STAGE_BYTES;      // two record buffers per expander warp
    const unsigned bar_full = smem_u32(&bars[0]), bar_empty = smem_u32(&bars[S]), bar_done = smem_u32(&bars[2 * S]);

    const unsigned int trow = task_row[task];
    const bool split = (trow >> 31) != 0;
    const int first_row = (int)(trow & 0x7fffffffu) - row_begin;
    int t0 = task_start[task], nt = task_start[task + 1] - t0;
    if (TSP_CHECKED)
    {
        // checked build: the task must lie inside the class's tiles and its 64 rows inside the caller's C
        const bool bad_task = t0 < 0 || nt < 0 || (long long)t0 + nt > bounds.tilenum, bad_rows = first_row < 0 || first_row + 64 > bounds.c_rows;
        if (bad_task || bad_rows)
        {
            if (tid == 0) atomicExch(err, bad_task ? 0x21 : 0x22);
            return;   // before any barrier or tensor-memory allocation
        }
    }

    // a slot is full when the B producers (PW warps, or the one TMA lane) and the tile's expander have arrived
    constexpr unsigned FULL_COUNT = (TMA ? 1 : PW * 32) + 1;
    if (tid == 0)
    {
        for (int s = 0; s < S; s++) { mbar_init(bar_full + 8 * s, FULL_COUNT); mbar_init(bar_empty + 8 * s, 1); }
        mbar_init(bar_done, 1);
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    if (warp == PW + NE)
    {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_u32(&tmem_slot)), "r"(C::TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
    const unsigned tmem_base = tmem_slot;
    bool ok = true;

    if (warp < PW)
    {
        // ------------------------------------------------------------ B producers
        if constexpr (TMA)
        {
            // one lane drives the copy engine: per tile one gather4 request per four gathered rows and 128-byte column
            // block; the bytes are counted on the slot's barrier
            if (warp == 0)
            {
                const int x0 = stripe * N;
                int idx_next = (nt > 0 && lane < C::BNK) ? __ldg(tile_colidx + (size_t)t0 * C::BNK + lane) : 0;
                for (int i = 0; i < nt && ok; i++)
                {
                    const int s = i % S;
                    if (i >= S) { ok = mbar_wait_warp(bar_empty + 8 * s, ((i / S) - 1) & 1, lane); if (!ok) break; }
                    const unsigned st = ring + s * C::STAGE_BYTES + C::A_BYTES, bar = bar_full + 8 * s;
                    int idx_cur = idx_next;
                    if (TSP_CHECKED && lane < C::BNK && (unsigned)idx_cur >= (unsigned)bounds.colA) { atomicExch(err, 0x20); idx_cur = 0; }
                    if (i + 1 < nt && lane < C::BNK) idx_next = __ldg(tile_colidx + (size_t)(t0 + i + 1) * C::BNK + lane);
                    if (lane == 0) mbar_expect_tx_only(bar, C::B_BYTES);
                    __syncwarp();
#pragma unroll
                    for (int g = 0; g < C::BNK / 4; g++)
                    {
                        const int r0 = __shfl_sync(0xffffffffu, idx_cur, 4 * g), r1 = __shfl_sync(0xffffffffu, idx_cur, 4 * g + 1);
                        const int r2 = __shfl_sync(0xffffffffu, idx_cur, 4 * g + 2), r3 = __shfl_sync(0xffffffffu, idx_cur, 4 * g + 3);
                        // rows 4g .. 4g+3 of the tile; for FP16 two groups share one 8-row atom
                        const unsigned atom = (unsigned)((g * 4) / C::ATOM_ROWS) * C::ATOM_BYTES + (unsigned)((g * 4) % C::ATOM_ROWS) * C::BOX_BYTES;
                        if (lane == 0)
                        {
#pragma unroll
                            for (int b = 0; b < C::NBOX; b++)
                                tma_gather4(st + (unsigned)b * C::KATOMS * C::ATOM_BYTES + atom, &bmap, x0 + b * C::BOX_COLS, r0, r1, r2, r3, bar);
                        }
                    }
                    if (lane == 0) mbar_arrive(bar);
                }
            }
        }
        else
        {
            // Chunk q = it*PW*32 + tid of a tile is 16-byte chunk c = tid % CPR of row k = it*KPI + tid/CPR, so the
            // source column offset and the swizzled destination of every copy are loop invariants.
            const unsigned ldb_b = (unsigned)ldb * C::SZ;
            const int c_mine = tid % C::CPR, k_mine = tid / C::CPR;
            const unsigned char *gsrc = dB + (size_t)stripe * C::RB + (size_t)c_mine * 16;
            const int *idx_ptr = tile_colidx + (size_t)t0 * C::BNK + k_mine;
            int cols_next[C::B_ITERS];
            unsigned dst_off[C::B_ITERS];
#pragma unroll
            for (int it = 0; it < C::B_ITERS; it++)
            {
                dst_off[it] = C::A_BYTES + b_chunk_offset<C>(it * C::KPI + k_mine, c_mine);
                cols_next[it] = nt > 0 ? __ldg(idx_ptr + it * C::KPI) : 0;
                if (TSP_CHECKED && (unsigned)cols_next[it] >= (unsigned)bounds.colA) { atomicExch(err, 0x20); cols_next[it] = 0; }
            }
            const unsigned long long pol_keep = policy_evict_last();
            // Nobody waits for the copies: every thread leaves an arrival on the slot's barrier that is delivered when its own
            // copies have landed, so every slot the MMA has released is in flight again at once.
            for (int i = 0; i < nt && ok; i++)
            {
                const int s = i % S;
                if (i >= S) { ok = mbar_wait_warp(bar_empty + 8 * s, ((i / S) - 1) & 1, lane); if (!ok) break; }
                const unsigned st = ring + s * C::STAGE_BYTES;
#pragma unroll
                for (int it = 0; it < C::B_ITERS; it++)
                    cp_async16_hint(st + dst_off[it], gsrc + (unsigned long long)(unsigned)cols_next[it] * ldb_b, pol_keep);
                cp_async_arrive(bar_full + 8 * s);
                idx_ptr += C::BNK;
                if (i + 1 < nt)
                {
#pragma unroll
                    for (int it = 0; it < C::B_ITERS; it++)
                    {
                        cols_next[it] = __ldg(idx_ptr + it * C::KPI);
                        if (TSP_CHECKED && (unsigned)cols_next[it] >= (unsigned)bounds.colA) { atomicExch(err, 0x20); cols_next[it] = 0; }
                    }
                }
            }
            asm volatile("cp.async.wait_all;\n" ::: "memory");   // no copy of this CTA outlives its shared memory
        }

        // ------------------------------------------------------------ epilogue (warps 0-3: tensor-memory quarter = warp)
        if (warp < 4)
        {
            if (ok && nt > 0)
            {
                ok = mbar_wait_warp(bar_done, 0, lane);
                asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
            }
            if (ok)
            {
                // with M = 64 the accumulator row r lives in tensor-memory lane (r/16)*32 + r%16
                const int quarter = warp & 3;
                const int row = quarter * 16 + (lane & 15);
                float *crow = dC + (size_t)(first_row + row) * (size_t)ldb + (size_t)stripe * N;
#pragma unroll 1
                for (int c0 = 0; c0 < N; c0 += 16)   // 16 columns at a time keeps the kernel within 40 registers (4 CTAs of 11 warps per SM)
                {
                    unsigned r[16];
                    if (nt > 0) tmem_ld16(tmem_base + ((unsigned)(quarter * 32) << 16) + (unsigned)c0, r);
                    else
                    {
#pragma unroll
                        for (int q = 0; q < 16; q++) r[q] = 0u;
                    }
                    if (lane < 16)
                    {
#pragma unroll
                        for (int q = 0; q < 16; q += 4)
                        {
                            if (split)
                                asm volatile("red.global.add.v4.f32 [%0], {%1,%2,%3,%4};\n" ::"l"(crow + c0 + q), "f"(__uint_as_float(r[q])),
                                             "f"(__uint_as_float(r[q + 1])), "f"(__uint_as_float(r[q + 2])), "f"(__uint_as_float(r[q + 3])) : "memory");
                            else
                                __stcs(reinterpret_cast<uint4 *>(crow + c0 + q), make_uint4(r[q], r[q + 1], r[q + 2], r[q + 3]));
                        }
                    }
                }
            }
        }
    }
    else if (warp < PW + NE)
    {
        // ------------------------------------------------------------ expanders: warp e owns tiles e, e+NE, ...
        const int e = warp - PW;
        const unsigned my_recs = recs + (unsigned)e * 2 * C::REC_BYTES;
        const int nte = nt > e ? (nt - e + NE - 1) / NE : 0;       // tiles of this expander
        // record words run two tiles ahead in registers, the record itself one tile ahead in shared memory
        unsigned w_cur = 0, w_cur_end = 0, w_next = 0, w_next_end = 0;
        auto load_words = [&](int i, unsigned &w, unsigned &w_end) {
            const unsigned rw = __ldg(rec_ptr + (size_t)t0 + i + (lane & 1));
            w = __shfl_sync(0xffffffffu, rw, 0);
            w_end = __shfl_sync(0xffffffffu, rw, 1) & 0x7fffffffu;
        };
        const unsigned long long pol_once = policy_evict_first();
        auto fetch_record = [&](unsigned w, unsigned w_end, int slot) {   // packed record -> private buffer (cp.async, caller commits)
            if (w >> 31) return;                                         // dense records go straight into the ring slot
            const unsigned chunks = min(w_end - w, (unsigned)C::REC_CHUNKS);
            const unsigned char *src = pack + (size_t)w * 16;
            for (unsigned q = lane; q < chunks; q += 32) cp_async16_hint(my_recs + (unsigned)slot * C::REC_BYTES + q * 16, src + (size_t)q * 16, pol_once);
        };
        if (nte > 0) { load_words(e, w_cur, w_cur_end); fetch_record(w_cur, w_cur_end, 0); }
        cp_async_commit();
        if (nte > 1) load_words(e + NE, w_next, w_next_end);
        for (int m = 0; m < nte; m++)
        {
            const int i = e + m * NE, s = i % S;
            // start the copy of the next record, then make sure this tile's record has landed
            unsigned w_next2 = 0, w_next2_end = 0;
            if (m + 1 < nte) fetch_record(w_next, w_next_end, (m + 1) & 1);
            cp_async_commit();
            if (m + 2 < nte) load_words(i + 2 * NE, w_next2, w_next2_end);
            cp_async_wait<1>();
            if (i >= S) { ok = mbar_wait_warp(bar_empty + 8 * s, ((i / S) - 1) & 1, lane); if (!ok) break; }
            const unsigned st = ring + s * C::STAGE_BYTES, bar = bar_full + 8 * s;
            if (w_cur >> 31)
            {
                if (lane == 0)   // a dense record goes from global memory straight into the A area; its bytes count on the slot's barrier
                {
                    mbar_expect_tx_only(bar, C::A_BYTES);
                    bulk_g2s(st, pack + (size_t)(w_cur & 0x7fffffffu) * 16, C::A_BYTES, bar);
                }
            }
            else expand_record<PREC>(my_recs + (unsigned)(m & 1) * C::REC_BYTES, min((w_cur_end - w_cur) * 16u / (2 + C::SZ), (unsigned)C::REC_MAX_VALS), st, lane);
            asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(bar);
            w_cur = w_next; w_cur_end = w_next_end; w_next = w_next2; w_next_end = w_next2_end;
        }
        cp_async_wait<0>();
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
            // the rows were written by cp.async (generic proxy), the tensor core reads them through the async proxy
            if (!TMA) asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
            asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
            const unsigned st = ring + s * C::STAGE_BYTES;
#pragma unroll
            for (int kk = 0; kk < 2; kk++)
            {
                // A: K-major, no swizzle; the two core-matrix columns of this K step are 1 KB apart,
                // 8-row groups 128 B apart
                const unsigned long long da = make_desc(st + kk * 2048, 1024, 128, 0);
                // B: MN-major; 64-column (128-byte) atoms KATOMS atoms apart, K atoms ATOM_BYTES apart
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
    if (warp == PW + NE)
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

template <int PREC, int N, bool TMA>
int launch64(tsp_handle *h, const void *d_b, float *d_c, int colB, cudaStream_t s)
{
    using C = Cfg64<PREC, N>;
    TspClass &c = h->cls[0];
    static bool configured[8] = {false};
    auto kern = k_spmm64<PREC, N, TMA>;
    if (!configured[h->device & 7])
    {
        TSP_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM));
        configured[h->device & 7] = true;
    }
    if (c.ntasks == 0) return TSP_OK;
    TspRange range("tsp 64-row class kernel");
    if (TMA && (h->bmap_ptr != d_b || h->bmap_cols != colB || h->bmap_box != C::BOX_COLS))   // the map depends on B's address and shape only
    {
        TSP_TRY(make_b_map(reinterpret_cast<CUtensorMap *>(h->bmap), PREC, d_b, h->colA, colB, C::BOX_COLS, C::BOX_BYTES));
        h->bmap_ptr = d_b; h->bmap_cols = colB; h->bmap_box = C::BOX_COLS;
    }
    dim3 grid(c.ntasks, colB / N);
    kern<<<grid, C::THREADS, C::SMEM, s>>>(*reinterpret_cast<const CUtensorMap *>(h->bmap), c.ntasks, colB, h->row_begin, c.d_task_row, c.d_task_start,
                                       c.d_tile_colidx, c.d_rec, c.d_pack, (const unsigned char *)d_b, d_c, h->d_error, tsp_bounds(h, 0));
    TSP_CUDA(cudaGetLastError());
    h->launches++;
    return TSP_OK;
}

template <int PREC, bool TMA>
int launch64_width(tsp_handle *h, const void *d_b, float *d_c, int colB, cudaStream_t s)
{
    switch (tsp_stripe_width(0, colB))
    {
    case 32: return launch64<PREC, 32, TMA>(h, d_b, d_c, colB, s);
    case 256: return launch64<PREC, 256, TMA>(h, d_b, d_c, colB, s);
    case 128: return launch64<PREC, 128, TMA>(h, d_b, d_c, colB, s);
    default: return launch64<PREC, 64, TMA>(h, d_b, d_c, colB, s);
    }
}

template <int PREC, int N>
void resources64(TspKernelResources *out)
{
    using C = Cfg64<PREC, N>;
    cudaFuncAttributes attr;
    memset(&attr, 0, sizeof(attr));
    cudaFuncGetAttributes(&attr, k_spmm64<PREC, N, false>);
    out->threads = C::THREADS;
    out->registers_per_thread = attr.numRegs;
    out->shared_bytes = C::SMEM + (long long)attr.sharedSizeBytes;
    out->tasks_per_block = 1;
    out->iteration_bytes = C::STAGE_BYTES;
}

}  // namespace

int tsp_launch_class64(tsp_handle *h, const void *d_b, float *d_c, int colB, cudaStream_t s)
{
    return h->precision == 0 ? launch64_width<0, false>(h, d_b, d_c, colB, s) : launch64_width<1, false>(h, d_b, d_c, colB, s);
}

int tsp_launch_class64_tma(tsp_handle *h, const void *d_b, float *d_c, int colB, cudaStream_t s)
{
    return h->precision == 0 ? launch64_width<0, true>(h, d_b, d_c, colB, s) : launch64_width<1, true>(h, d_b, d_c, colB, s);
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
