// SpMM kernel for the 64-row tile class: tcgen05.mma with the accumulator in tensor memory (sm_100a), fed from
// PACKED tiles.
//
// Replaces upstream stir_spmm_cuda_kernel_v64* (src/tilespmm_cuda.h:1025-1632) and switch_tilespmm_cuda_v64
// (src/tilespmm_cuda.h:1710-1744).  Upstream keeps every 64-row tile as a dense, zero-padded 4 KB block
// (src/csr2tile.h:309-373); on a stencil 95% of those bytes are zeros.  Here a tile is a RECORD in one byte array:
//   packed record   64 row masks (bit k of mask r: position (r, k) holds an entry; 16-bit masks for TF32 tiles of
//                   16 columns, 32-bit masks for FP16 tiles of 32 columns) followed by the values of the set
//                   positions in row-major order, padded to 16 bytes -- for tiles with at most REC_MAX_VALS values;
//   dense record    the 4 KB tile in the K-major core-matrix order tcgen05.mma reads -- for fuller tiles.
// rec[t] is the record's offset in 16-byte units, bit 31 set for a dense record.
//
// One CTA owns one task (a 64-row panel or a slice of a split panel) and one column stripe of up to 256 columns, so
// the tile records and column indices are read once per 256 columns (upstream: once per 64).  Roles:
//   warps 0-3  producers.  Warp w owns tiles w, w+4, ... of the task.  For its tile it (1) gathers the B rows named by
//              tile_colidx into the ring slot in the swizzled MN-major operand layout -- 16-byte cp.async, one gathered
//              row segment per warp instruction, or, in the TMA form, cp.async.bulk.tensor ... tile::gather4 requests
//              issued by one lane; (2) prefetches the record of its NEXT tile into a private buffer; (3) expands the
//              record of the current tile into the slot's 4 KB A area in operand order (zero fill + one store per
//              value), or starts one 4 KB bulk copy for a dense record; (4) publishes the slot on its mbarrier.
//              Afterwards the four warps are the epilogue: tcgen05.ld of the 64 x N FP32 accumulator -> C.
//   warp 4     allocates tensor memory; one lane issues two tcgen05.mma (M=64, N=stripe, K=16 FP16 / K=8 TF32) per
//              tile and releases ring slots with tcgen05.commit.
// The accumulator of a whole task stays in tensor memory (64 lanes x N columns) and is written once, with vector
// stores, or vector red.global.add for the slices of a split panel.
// Every wait on an mbarrier is bounded; when one runs out the kernel records it in *err, frees its tensor memory and
// returns.
#include <cuda.h>

#include "tsp_internal.cuh"

namespace
{

constexpr unsigned WAIT_LIMIT = 1u << 22;
constexpr int PW = 4;                  // producer (and epilogue) warps
constexpr int THREADS = (PW + 1) * 32;

#ifndef TSP64_DEPTH
#define TSP64_DEPTH 2                  // tiles a producer warp keeps in flight (1 or 2)
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
    static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
    static constexpr int ITERS = BNK * CPR / 32;              // warp-wide copies per tile
    static constexpr int DEPTH = TSP64_DEPTH;
#ifdef TSP64_STAGES
    static constexpr int STAGES = TSP64_STAGES;
#else
    static constexpr int STAGES = N == 256 ? 5 : (N == 128 ? (DEPTH == 2 ? 8 : 5) : 8);
#endif
    static_assert(STAGES > PW, "a producer warp may wait for the slot of its next tile while its previous tile is unpublished");
    // packed records
    static constexpr int MASK_BYTES = 64 * BNK / 8;           // 128 (TF32) / 256 (FP16)
    static constexpr int REC_MAX_VALS = TSP_REC_MAX_VALS(PREC);
    static constexpr int REC_BYTES = MASK_BYTES + REC_MAX_VALS * SZ;
    static constexpr int REC_CHUNKS = REC_BYTES / 16;
    static constexpr int SMEM = STAGES * STAGE_BYTES + PW * 2 * REC_BYTES + 1024;  // + slack to align the ring to 1 KB
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

// Expands the packed record at shared address `rec` into the 4 KB A area at shared address `a` (K-major core
// matrices, tsp_umma_index): zero fill, then one store per value.  Lane l owns rows 2l and 2l+1, whose values are
// contiguous in the record, so the position of a lane's first value is the prefix sum of the lanes' entry counts.
template <int PREC>
__device__ __forceinline__ void expand_record(unsigned rec, unsigned a, int lane)
{
    __syncwarp();   // the record was copied in by all lanes of the warp
    const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
    for (int q = 0; q < 8; q++)
        asm volatile("st.shared.v4.b32 [%0], {%1,%2,%3,%4};\n" ::"r"(a + (unsigned)(q * 32 + lane) * 16), "r"(zero.x), "r"(zero.y), "r"(zero.z), "r"(zero.w) : "memory");
    unsigned w0, w1;
    if constexpr (PREC == 1)
    {
        unsigned w;
        asm volatile("ld.shared.b32 %0, [%1];\n" : "=r"(w) : "r"(rec + (unsigned)lane * 4));
        w0 = w & 0xffffu; w1 = w >> 16;
    }
    else
        asm volatile("ld.shared.v2.b32 {%0,%1}, [%2];\n" : "=r"(w0), "=r"(w1) : "r"(rec + (unsigned)lane * 8));
    const int cnt = __popc(w0) + __popc(w1);
    int incl = cnt;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) { const int y = __shfl_up_sync(0xffffffffu, incl, o); if (lane >= o) incl += y; }
    __syncwarp();   // the zero fill of every lane is ordered before any lane's value stores
    constexpr int SZ = PREC == 0 ? 2 : 4, T = 16 / SZ, MASKS = PREC == 0 ? 256 : 128;
    unsigned src = rec + MASKS + (unsigned)(incl - cnt) * SZ;
#pragma unroll
    for (int half = 0; half < 2; half++)
    {
        unsigned w = half ? w1 : w0;
        const int r = 2 * lane + half;
        const unsigned row_off = a + (unsigned)(r >> 3) * 128 + (unsigned)(r & 7) * 16;
        while (w)
        {
            const int k = __ffs(w) - 1;
            w &= w - 1;
            const unsigned dst = row_off + (unsigned)(k / T) * 1024 + (unsigned)(k % T) * SZ;
            if constexpr (PREC == 1)
            {
                unsigned v;
                asm volatile("ld.shared.b32 %0, [%1];\n" : "=r"(v) : "r"(src));
                asm volatile("st.shared.b32 [%0], %1;\n" ::"r"(dst), "r"(v) : "memory");
            }
            else
            {
                unsigned short v;
                asm volatile("ld.shared.b16 %0, [%1];\n" : "=h"(v) : "r"(src));
                asm volatile("st.shared.b16 [%0], %1;\n" ::"r"(dst), "h"(v) : "memory");
            }
            src += SZ;
        }
    }
}

template <int PREC, int N, bool TMA>
__global__ void __launch_bounds__(THREADS)
k_spmm64(const __grid_constant__ CUtensorMap bmap, int ntasks, int ldb, int row_begin, const unsigned int *__restrict__ task_row,
         const int *__restrict__ task_start, const int *__restrict__ tile_colidx, const unsigned int *__restrict__ rec_ptr,
         const unsigned char *__restrict__ pack, const unsigned char *__restrict__ dB, float *__restrict__ dC, int *__restrict__ err)
{
    using C = Cfg64<PREC, N>;
    constexpr int S = C::STAGES, D = C::DEPTH;
    extern __shared__ unsigned char smem_raw[];
    __shared__ __align__(8) unsigned long long bars[2 * C::STAGES + 1];
    __shared__ unsigned tmem_slot;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, tid = threadIdx.x;
    const int task = blockIdx.x, stripe = blockIdx.y;
    const unsigned ring = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const unsigned recs = ring + S * C::STAGE_BYTES;      // 2 record buffers per producer warp
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
    if (warp == PW)
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
        // ------------------------------------------------------------ producers: warp w owns tiles w, w+PW, ...
        const unsigned ldb_b = (unsigned)ldb * C::SZ;
        const unsigned my_recs = recs + (unsigned)warp * 2 * C::REC_BYTES;
        const int ntw = nt > warp ? (nt - warp + PW - 1) / PW : 0;     // tiles of this warp
        // lane constants of the gather: copy q = it*32 + lane of a tile is chunk c = q % CPR of row k = q / CPR
        const int c_lane = C::CPR >= 32 ? lane : lane % C::CPR, k_lane = C::CPR >= 32 ? 0 : lane / C::CPR;
        const unsigned char *gsrc = dB + (size_t)stripe * C::RB + (size_t)c_lane * 16;

        // state of the tile that will be issued next: its column indices (lane k: row k) and record word
        int idx_next = 0;
        unsigned rec_next = 0, rec_next_end = 0;
        auto fetch_meta = [&](int i) {   // i: tile index within the task
            const size_t t = (size_t)t0 + i;
            if (lane < C::BNK) idx_next = __ldg(tile_colidx + t * C::BNK + lane);
            const unsigned rw = __ldg(rec_ptr + t + (lane & 1));
            rec_next = __shfl_sync(0xffffffffu, rw, 0);
            rec_next_end = __shfl_sync(0xffffffffu, rw, 1) & 0x7fffffffu;
        };
        auto fetch_record = [&](int slot) {   // packed record of the "next" tile -> private buffer `slot` (cp.async, caller commits)
            if (rec_next >> 31) return;       // dense records go straight into the ring slot
            const unsigned chunks = min(rec_next_end - (rec_next & 0x7fffffffu), (unsigned)C::REC_CHUNKS);
            const unsigned char *src = pack + (size_t)(rec_next & 0x7fffffffu) * 16;
            for (unsigned q = lane; q < chunks; q += 32) cp_async16(my_recs + (unsigned)slot * C::REC_BYTES + q * 16, src + (size_t)q * 16);
        };
        if (ntw > 0)
        {
            fetch_meta(warp);
            fetch_record(0);
        }
        cp_async_commit();
        if (D == 1) cp_async_wait<0>();

        auto publish = [&](int i) {  // tile i is complete in shared memory: hand it to the MMA warp
            asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_full + 8 * (i % S));
        };

        for (int j = 0; j < ntw; j++)
        {
            const int i = warp + j * PW, s = i % S;
            if (i >= S) { ok = mbar_wait_warp(bar_empty + 8 * s, ((i / S) - 1) & 1, lane); if (!ok) break; }
            const unsigned st = ring + s * C::STAGE_BYTES, bar = bar_full + 8 * s;
            const int idx_cur = idx_next;
            const unsigned rec_cur = rec_next;
            const bool dense = (rec_cur >> 31) != 0;
            // ---- B rows of tile i
            if constexpr (TMA)
            {
                if (lane == 0) mbar_expect_tx_only(bar, C::B_BYTES + (dense ? C::A_BYTES : 0));
                __syncwarp();
                const int x0 = stripe * N;
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
                            tma_gather4(st + C::A_BYTES + (unsigned)b * C::KATOMS * C::ATOM_BYTES + atom, &bmap, x0 + b * C::BOX_COLS, r0, r1, r2, r3, bar);
                    }
                }
            }
            else
            {
                if (dense && lane == 0) mbar_expect_tx_only(bar, C::A_BYTES);
#pragma unroll
                for (int it = 0; it < C::ITERS; it++)
                {
                    const int k = C::CPR >= 32 ? it / (C::CPR / 32) : it * (32 / C::CPR) + k_lane;
                    const int c = C::CPR >= 32 ? (it % (C::CPR / 32)) * 32 + c_lane : c_lane;
                    const int col = __shfl_sync(0xffffffffu, idx_cur, k);
                    const size_t extra = C::CPR > 32 ? (size_t)(it % (C::CPR / 32)) * 512 : 0;
                    cp_async16(st + C::A_BYTES + b_chunk_offset<C>(k, c), gsrc + extra + (unsigned long long)(unsigned)col * ldb_b);
                }
            }
            if (dense && lane == 0) bulk_g2s(st, pack + (size_t)(rec_cur & 0x7fffffffu) * 16, C::A_BYTES, bar);
            // ---- record and indices of this warp's next tile
            if (j + 1 < ntw)
            {
                fetch_meta(i + PW);
                fetch_record((j + 1) & 1);
            }
            cp_async_commit();
            if (D == 2) cp_async_wait<1>();     // everything up to the previous iteration's group has landed
            // ---- A of tile i
            if (!dense) expand_record<PREC>(my_recs + (unsigned)(j & 1) * C::REC_BYTES, st, lane);
            if (D == 1) { cp_async_wait<0>(); publish(i); }
            else if (j > 0) publish(i - PW);
        }
        cp_async_wait<0>();
        if (D == 2 && ok && ntw > 0) publish(warp + (ntw - 1) * PW);

        // ------------------------------------------------------------ epilogue
        if (ok && nt > 0)
        {
            ok = mbar_wait_warp(bar_done, 0, lane);
            asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
        }
        if (ok)
        {
            // with M = 64 the accumulator row r lives in tensor-memory lane (r/16)*32 + r%16; a warp reads the 32 lanes
            // of its quarter (warp % 4)
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
                    for (int q = 0; q < 32; q++) r[q] = 0u;
                }
                if (lane < 16)
                {
#pragma unroll
                    for (int q = 0; q < 32; q += 4)
                    {
                        if (split)
                            asm volatile("red.global.add.v4.f32 [%0], {%1,%2,%3,%4};\n" ::"l"(crow + c0 + q), "f"(__uint_as_float(r[q])),
                                         "f"(__uint_as_float(r[q + 1])), "f"(__uint_as_float(r[q + 2])), "f"(__uint_as_float(r[q + 3])) : "memory");
                        else
                            *reinterpret_cast<uint4 *>(crow + c0 + q) = make_uint4(r[q], r[q + 1], r[q + 2], r[q + 3]);
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
    if (warp == PW)
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
    if (TMA && (h->bmap_ptr != d_b || h->bmap_cols != colB || h->bmap_box != C::BOX_COLS))   // the map depends on B's address and shape only
    {
        TSP_TRY(make_b_map(reinterpret_cast<CUtensorMap *>(h->bmap), PREC, d_b, h->colA, colB, C::BOX_COLS, C::BOX_BYTES));
        h->bmap_ptr = d_b; h->bmap_cols = colB; h->bmap_box = C::BOX_COLS;
    }
    dim3 grid(c.ntasks, colB / N);
    kern<<<grid, THREADS, C::SMEM, s>>>(*reinterpret_cast<const CUtensorMap *>(h->bmap), c.ntasks, colB, h->row_begin, c.d_task_row, c.d_task_start,
                                       c.d_tile_colidx, c.d_rec, c.d_pack, (const unsigned char *)d_b, d_c, h->d_error);
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
    out->threads = THREADS;
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
