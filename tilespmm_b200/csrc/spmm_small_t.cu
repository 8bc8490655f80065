// SpMM kernel for the 16-row and 8-row tile classes on tcgen05.mma, transposed form (sm_100a).
//
// Same job as upstream stir_spmm_cuda_kernel_v16*/v8* (src/tilespmm_cuda.h:12-1023), different mapping: the
// product is computed as C^T, so that the GATHERED rows of B are the large operand of the MMA.  For one tile
//     D[m][n] += sum_k Bg[k][m] * Atile[n][k]     m: column of the stripe (M = 128 or 64)
//                                                 n: row of the panel   (N = 16; an 8-row panel uses half)
//                                                 k: column of the tile (K = 16 FP16 / 8 TF32, one MMA)
// The gathered rows go from global memory straight into the swizzled MN-major operand layout with 16-byte
// cp.async and are read from shared memory by the tensor core only: no ld.shared, no register fragments, and the
// accumulator (128 lanes x 16 columns) lives in tensor memory, two of them so that the epilogue of one task
// overlaps the gathers and MMAs of the next.
//
// The kernel is persistent: CTA b works on units (task, stripe) b, b + gridDim.x, ...  Roles (11 warps):
//   warp 10    index warp: walks the CTA's units ahead of everybody else and turns them into a stream of groups of
//              up to G tiles of one unit: a descriptor plus the tiles' column indices, in a ring 16 groups deep.
//   warps 0-3  producers: warp w fetches groups w, w+4, ... on its own.  Per tile 4 KB (2 KB for 64-column stripes)
//              of gathered rows plus the tile's values, which upstream's fragment order stores as a 32 x W word
//              matrix and the K-major core-matrix operand layout wants transposed (W x 32): W 4-byte cp.async per
//              lane do that on the fly.  Nobody waits for data: each lane leaves a cp.async.mbarrier.arrive on the
//              slot's full barrier, which fires when its copies have landed.
//   warps 4-5  MMA issuers, one lane each: the chain wait -> tcgen05.mma (one per tile) -> tcgen05.commit is latency
//              bound, so two lanes share it; issuer m takes every second unit and owns accumulator m.
//   warps 6-9  epilogue: tcgen05.ld of the accumulator quarter of the warp, then one 128-byte row segment per
//              store instruction (red.global.add for the slices of a split panel).
// Every wait is bounded; when one runs out the role records which in *err and leaves its loop.
//
// Measured on B200 (27-point stencil 64^3, TF32, 128 columns, 8-row tiles): 0.134 ms against 0.130 ms of the
// mma.sync kernel in spmm_small.cu; on R-MAT matrices, whose units are one or two tiles long, it is slower (0.66 ms
// against 0.45 ms), because a unit costs an accumulator hand-over however short it is.  Both kernels sit at the
// rate at which an SM can gather 512-byte rows from L2 (about 14.5 TB/s over the chip for a 134 MB operand), so this
// kernel is kept as an option (environment TSP_SMALL=t) and the default stays with spmm_small.cu.
#include "tsp_internal.cuh"

namespace
{

constexpr long long WAIT_CYCLES = 1ll << 28;   // ~0.15 s: far beyond any wait of a healthy run
constexpr int PW = 4;                         // producer warps 0-3
constexpr int W_MMA = 4, NMMA = 2;            // warps 4-5: MMA issuers (one lane each), one per accumulator
constexpr int W_EPI = W_MMA + NMMA;           // warps 6-9: epilogue
constexpr int W_INDEX = W_EPI + 4;            // warp 10: index warp
constexpr int THREADS = (W_INDEX + 1) * 32;
constexpr int CTAS = 3;                       // resident CTAs per SM the kernel is compiled for (registers: 352 threads)

template <int PREC, int CLS, int NS>
struct CfgT
{
    static constexpr int SZ = PREC == 0 ? 2 : 4;
    static constexpr int BM = CLS == 1 ? 16 : 8;
    static constexpr int BN = PREC == 0 ? 16 : 8;          // K extent of a tile = one MMA
    static constexpr int RB = NS * SZ;                     // bytes of one gathered row segment
    static constexpr int CPR = RB / 16;                    // 16-byte chunks per row
    static constexpr int GB = BN * RB;                     // gathered bytes per tile: 4096 (NS 128) / 2048 (NS 64)
    static constexpr int A_BYTES = BM * BN * SZ;           // 512 (16-row) / 256 (8-row)
    static constexpr int A_SLOT = 512;                     // an 8-row tile leaves the upper half unused (see MMA)
    static constexpr int AW = A_BYTES / 128;               // words per lane of the fragment-order tile (4 / 2)
    static constexpr int G = 4;                            // tiles per ring slot (one hand-over per group of G tiles)
    static constexpr int STAGE_BYTES = G * (GB + A_SLOT);
    static constexpr int STAGES = 4;                       // one slot per producer warp
    static constexpr int R = 16;                           // depth of the descriptor / column-index ring (groups)
    static constexpr int IDX_BYTES = R * G * BN * 4;
    static constexpr int NBARS = 2 * STAGES + 4 + 2 * R;
    static constexpr int RING_BYTES = STAGES * STAGE_BYTES;
    static constexpr int SMEM = RING_BYTES + IDX_BYTES + R * 8 + NBARS * 8 + 16;
    // MN-major operand layout of the gathered rows, as in the 64-row kernel: FP16 128-byte swizzle (atoms of
    // 8 K-rows x 128 B), TF32 128-byte swizzle with 32-byte atomicity (atoms of 4 K-rows x 128 B); a tile is
    // two atoms deep in K
    static constexpr int MODE = PREC == 1 ? 1 : 2;
    static constexpr int ATOM_BYTES = PREC == 1 ? 512 : 1024;
    static constexpr int KPI = CPR >= 32 ? 1 : 32 / CPR;   // tile rows covered by one warp-wide copy
    static constexpr int B_ITERS = BN / KPI;               // warp-wide copies per tile (8 or 4)
    static constexpr int IDXV = (G * BN + 31) / 32;        // registers per lane that hold a group's column indices
    static constexpr int TMEM_COLS = 32;                   // two accumulators of 16 columns
    static_assert(B_ITERS >= 1 && BN % KPI == 0, "producer mapping");
    // tcgen05.alloc blocks until columns are free, so the CTAs that can be resident on an SM together (bounded by the
    // 2048 threads of an SM) must never ask for more than the 512 columns of its tensor memory
    static_assert((2048 / THREADS) * TMEM_COLS <= 512, "resident CTAs would oversubscribe tensor memory");
    // A parity wait on an mbarrier is only meaningful for a waiter that is neither two phases ahead of the barrier nor
    // two behind.  Every barrier here therefore has one waiting agent that takes each phase in turn: with R % PW == 0
    // and STAGES % PW == 0 a descriptor slot and a data slot always belong to the same producer warp (the MMA issuers
    // release data slots out of order, so "some producer warp" would not do).  The full barriers, which the two
    // issuers share, are covered by the issuers' own hand-over (front[] in the kernel).
    static_assert(G <= 15 && STAGES % PW == 0 && R % PW == 0, "pipeline depths");
    static_assert(STAGE_BYTES % 1024 == 0 && GB % 1024 == 0, "the swizzled operand tiles must start on 1 KB boundaries");
};

__device__ __forceinline__ unsigned smem_u32(const void *p) { return (unsigned)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void cp_async16(unsigned smem, const void *gmem)
{
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(smem), "l"(gmem));
}
__device__ __forceinline__ void cp_async4(unsigned smem, const void *gmem)
{
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;\n" ::"r"(smem), "l"(gmem));
}
__device__ __forceinline__ void mbar_init(unsigned bar, unsigned count) { asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(bar), "r"(count)); }
// arrive on the mbarrier when every cp.async this thread has issued so far has landed; the thread itself does not wait
__device__ __forceinline__ void cp_async_arrive(unsigned bar)
{
    asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];\n" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive(unsigned bar) { asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(bar) : "memory"); }
__device__ __forceinline__ bool mbar_wait(unsigned bar, unsigned parity)
{
    {
        unsigned done;   // fast path: no suspension when the phase is already complete
        asm volatile("{\n\t.reg .pred p;\n\tmbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}\n"
                     : "=r"(done) : "r"(bar), "r"(parity) : "memory");
        if (done) return true;
    }
    const long long t_start = clock64();
    for (;;)
    {
        unsigned done;
        asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}\n"
                     : "=r"(done) : "r"(bar), "r"(parity) : "memory");
        if (done) return true;
        if (clock64() - t_start > WAIT_CYCLES) return false;
    }
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
__device__ __forceinline__ void tmem_ld16(unsigned taddr, unsigned (&r)[16])
{
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
                   "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
                 : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
}
__device__ __forceinline__ void tmem_ld8(unsigned taddr, unsigned (&r)[16])
{
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
                 : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
}


// tile range and stripe of unit u (units past the end are empty)
struct Unit
{
    int t0, t1, stripe, task;
};
__device__ __forceinline__ Unit load_unit(long long u, long long nunits, int nstripes, const int *__restrict__ task_start)
{
    Unit r;
    if (u >= nunits) { r.t0 = r.t1 = 0; r.stripe = 0; r.task = 0; return r; }
    // units fit 32 bits (the launcher checks), which keeps 64-bit division out of the per-unit path
    r.task = (int)((unsigned)u / (unsigned)nstripes);
    r.stripe = (int)((unsigned)u - (unsigned)r.task * (unsigned)nstripes);
    r.t0 = __ldg(task_start + r.task);
    r.t1 = __ldg(task_start + r.task + 1);
    return r;
}

// group descriptor: {first tile, tiles (bits 0-3) | stripe (bits 8-23) | end of stream (bit 31)}
constexpr unsigned D_END = 1u << 31;

template <int PREC, int CLS, int NS>
__global__ void __launch_bounds__(THREADS, CTAS)
k_spmm_small_t(int ntasks, int nstripes, int ldb /* elements */, int row_begin, const unsigned int *__restrict__ task_row,
               const int *__restrict__ task_start, const int *__restrict__ tile_colidx, const unsigned char *__restrict__ tile_val,
               const unsigned char *__restrict__ dB, float *__restrict__ dC, int *__restrict__ err)
{
    using C = CfgT<PREC, CLS, NS>;
    constexpr int S = C::STAGES, G = C::G, R = C::R;
    // all shared memory is dynamic, so that the ring starts at offset 0 of the CTA's window (1 KB aligned, which the
    // swizzled operand layouts need) and four CTAs fit an SM: ring | column-index ring | descriptors | mbarriers | slot
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    int(*idx_ring)[G * C::BN] = reinterpret_cast<int(*)[G * C::BN]>(smem_raw + C::RING_BYTES);
    uint2 *desc_ring = reinterpret_cast<uint2 *>(smem_raw + C::RING_BYTES + C::IDX_BYTES);
    unsigned long long *bars = reinterpret_cast<unsigned long long *>(smem_raw + C::RING_BYTES + C::IDX_BYTES + R * 8);
    unsigned &tmem_slot = *reinterpret_cast<unsigned *>(smem_raw + C::RING_BYTES + C::IDX_BYTES + R * 8 + C::NBARS * 8);
    // front[m]: index of the next group MMA issuer m will wait for (it is past the full barrier of all its earlier groups)
    volatile int *front = reinterpret_cast<volatile int *>(smem_raw + C::RING_BYTES + C::IDX_BYTES + R * 8 + C::NBARS * 8 + 4);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, tid = threadIdx.x;
    const unsigned ring = smem_u32(smem_raw);
    if (ring & 1023u)
    {
        if (tid == 0) atomicExch(err, 4);
        return;
    }
    const unsigned bar_full = smem_u32(&bars[0]), bar_empty = smem_u32(&bars[S]);
    const unsigned bar_acc_full = smem_u32(&bars[2 * S]), bar_acc_empty = smem_u32(&bars[2 * S + 2]);
    const unsigned bar_desc_full = smem_u32(&bars[2 * S + 4]), bar_desc_empty = smem_u32(&bars[2 * S + 4 + R]);
    const long long nunits = (long long)ntasks * nstripes, stride = gridDim.x;

    if (tid == 0)
    {
        for (int s = 0; s < S; s++) { mbar_init(bar_full + 8 * s, 32); mbar_init(bar_empty + 8 * s, 1); }
        for (int b = 0; b < 2; b++) { mbar_init(bar_acc_full + 8 * b, 1); mbar_init(bar_acc_empty + 8 * b, 4); }
        front[0] = front[1] = 0;
        for (int r = 0; r < R; r++) { mbar_init(bar_desc_full + 8 * r, 33); mbar_init(bar_desc_empty + 8 * r, 1); }
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    if (warp == W_MMA)
    {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_u32(&tmem_slot)), "r"(C::TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
    const unsigned tmem_base = tmem_slot;
    bool ok = true;
    int fail = 0;   // which wait gave up (reported through *err as 0x100 + code)

    if (warp == W_INDEX)
    {
        // ------------------------------------------------------------ index warp
        // Walks the units of this CTA ahead of everybody else and turns them into a stream of groups: a descriptor
        // (first tile, tile count, flags, stripe) plus the column indices of the group's tiles, copied into a ring
        // R groups deep.  Producers and the MMA lane only read that ring, so no global load sits in their loops.
        long long u = blockIdx.x;
        Unit cur = load_unit(u, nunits, nstripes, task_start);
        Unit nxt = load_unit(u + stride, nunits, nstripes, task_start);
        int x = 0;
        int ends_sent = 0;   // every producer warp takes every PW-th group, so each gets its own end marker
        while (ends_sent < PW && ok)
        {
            // next group: [t, t + cnt) of unit cur, or the end marker
            while (u < nunits && cur.t0 == cur.t1)
            {
                // empty from the start or used up (t0 advances through the unit)
                u += stride; cur = nxt;
                nxt = load_unit(u + stride, nunits, nstripes, task_start);
            }
            const bool end = u >= nunits;
            const int slot = x % R;
            if (x >= R) ok = __all_sync(0xffffffffu, mbar_wait(bar_desc_empty + 8 * slot, ((x / R) - 1) & 1));
            if (!ok) fail = 1;
            if (!ok) break;
            if (end)
            {
                if (lane == 0) desc_ring[slot] = make_uint2(0u, D_END);
                ends_sent++;
            }
            else
            {
                const int left = cur.t1 - cur.t0;
                const int cnt = left < G ? left : G;
                if (lane == 0)
                    desc_ring[slot] = make_uint2((unsigned)cur.t0, (unsigned)cnt | ((unsigned)cur.stripe << 8));
                if (lane * 4 < cnt * C::BN)
                    cp_async16(smem_u32(&idx_ring[slot][lane * 4]), tile_colidx + (size_t)cur.t0 * C::BN + lane * 4);
                cur.t0 += cnt;
            }
            // the slot is announced by 33 arrivals: one per lane, delivered when that lane's copies have landed (the
            // lane does not wait), and lane 0's own, which publishes the descriptor it stored
            cp_async_arrive(bar_desc_full + 8 * slot);
            if (lane == 0) mbar_arrive(bar_desc_full + 8 * slot);
            x++;
        }
        asm volatile("cp.async.wait_all;\n" ::: "memory");
    }
    else if (warp < PW)
    {
        // ------------------------------------------------------------ producers
        // Producer warp w fetches groups w, w + PW, ... on its own, so the fixed costs of a group (descriptor, slot
        // wait) of one warp hide behind the copies of the other three.  Warp-wide copy `it` of a tile moves 16-byte
        // chunk c = lane % CPR of rows k = it*KPI + lane/CPR: the source column offset and the swizzled destination
        // of every copy are loop invariants.
        const unsigned ldb_b = (unsigned)ldb * C::SZ;
        const int c_mine = lane % C::CPR, k_mine = lane / C::CPR;
        unsigned dst_off[C::B_ITERS];
#pragma unroll
        for (int it = 0; it < C::B_ITERS; it++)
        {
            const int k = it * C::KPI + k_mine, c = c_mine;
            if (C::MODE == 2) { const int ka = k >> 3, kr = k & 7; dst_off[it] = ((c >> 3) * 2 + ka) * 1024 + kr * 128 + (((c & 7) ^ kr) << 4); }
            else { const int ka = k >> 2, kr = k & 3; dst_off[it] = ((c >> 3) * 2 + ka) * 512 + kr * 128 + (((((c & 7) >> 1) ^ kr) << 5) | ((c & 1) << 4)); }
        }
        // values: lane l of the fragment-order tile owns words l*AW .. l*AW + AW-1; word j goes to row j, word l
        const unsigned char *gbase = dB + (size_t)c_mine * 16;
        for (int gi = warp; ok; gi += PW)
        {
            const int slot = gi % R;
            ok = __all_sync(0xffffffffu, mbar_wait(bar_desc_full + 8 * slot, (gi / R) & 1));
            if (!ok) fail = 2;
            if (!ok) break;
            const uint2 d = desc_ring[slot];
            if (d.y & D_END) break;
            const int cnt = (int)(d.y & 15u);
            int idxv[C::IDXV];   // column index q of the group in lane q % 32 of register q / 32
#pragma unroll
            for (int q = 0; q < C::IDXV; q++) idxv[q] = (q * 32 + lane < G * C::BN) ? idx_ring[slot][q * 32 + lane] : 0;
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_desc_empty + 8 * slot);

            const int s = gi % S;
            // slot s is always refilled by this warp (STAGES % PW == 0), which has seen every earlier release of it
            if (gi >= S) { ok = __all_sync(0xffffffffu, mbar_wait(bar_empty + 8 * s, ((gi / S) - 1) & 1)); if (!ok) fail = 3; }
            if (!ok) break;
            const unsigned st = ring + s * C::STAGE_BYTES;
            const unsigned char *gsrc = gbase + (size_t)((d.y >> 8) & 0xffffu) * C::RB;
            const unsigned char *asrc = tile_val + (size_t)d.x * C::A_BYTES + lane * (C::AW * 4);
#pragma unroll
            for (int j = 0; j < G; j++)
            {
                if (j < cnt)
                {
#pragma unroll
                    for (int w = 0; w < C::AW; w++)
                        cp_async4(st + G * C::GB + j * C::A_SLOT + w * 128 + lane * 4, asrc + (size_t)j * C::A_BYTES + w * 4);
#pragma unroll
                    for (int it = 0; it < C::B_ITERS; it++)
                    {
                        const int q = j * C::BN + it * C::KPI + k_mine;
                        const int col = __shfl_sync(0xffffffffu, idxv[q / 32], q % 32);
                        cp_async16(st + j * C::GB + dst_off[it], gsrc + (unsigned long long)(unsigned)col * ldb_b);
                    }
                }
            }
            // the slot's full barrier takes one arrival per lane, delivered when that lane's copies have landed: nobody
            // waits for data here, so every slot the MMA has released is in flight
            cp_async_arrive(bar_full + 8 * s);
        }
        asm volatile("cp.async.wait_all;\n" ::: "memory");
    }
    else if (warp < W_EPI)
    {
        // ------------------------------------------------------------ MMA issuers
        // The chain wait -> tcgen05.mma -> commit of one thread is latency bound (a few hundred cycles per group), so
        // two lanes share it: issuer m takes every second unit with tiles and owns accumulator m.
        if (lane == 0)
        {
            const int me = warp - W_MMA;
            // instruction descriptor: D = F32, A/B = F16 or TF32, A (gathered rows) MN-major, B (tile values) K-major,
            // N = 16, M = stripe width
            const unsigned fmt = PREC == 0 ? 0u : 2u;
            const unsigned idesc = (1u << 4) | (fmt << 7) | (fmt << 10) | (1u << 15) | (0u << 16) | ((16u >> 3) << 17) | ((unsigned)(NS >> 4) << 24);
            // The lane walks the units itself (ranges fetched one unit ahead) and cuts them into the same groups as the
            // index warp, so the only waits in its loop are the slot's full barrier and, per unit, the accumulator.
            long long u = blockIdx.x;
            Unit cur = load_unit(u, nunits, nstripes, task_start);
            Unit nxt = load_unit(u + stride, nunits, nstripes, task_start);
            int acc_it = 0, gi = 0;
            while (u < nunits && ok)
            {
                const int nt = cur.t1 - cur.t0;
                if (nt > 0 && (acc_it & 1) != me)
                {
                    gi += (nt + G - 1) / G;   // the other issuer's unit
                    acc_it++;
                }
                else if (nt > 0)
                {
                    const int buf = acc_it & 1, g0 = gi;
                    front[me] = g0;
                    // the epilogue must have drained this accumulator (two units ago)
                    if (acc_it >= 2) ok = mbar_wait(bar_acc_empty + 8 * buf, ((acc_it >> 1) - 1) & 1);
                    if (!ok) fail = 4;
                    if (!ok) break;
                    const unsigned tmem_d = tmem_base + (unsigned)(buf * 16);
                    unsigned accumulate = 0;
                    for (int i = 0; i < nt; i += G, gi++)
                    {
                        const int s = gi % S;
                        // A wait on a phase parity is only meaningful when the slot's previous phase is known to be
                        // complete.  This lane saw that itself when group gi - S was its own; when it was the other
                        // issuer's, wait until that lane reports to be past it.
                        if (gi - S >= 0 && gi - S < g0)
                        {
                            const long long t_start = clock64();
                            while (front[me ^ 1] <= gi - S)
                                if (clock64() - t_start > WAIT_CYCLES) { ok = false; fail = 5; break; }
                            if (!ok) break;
                        }
                        ok = mbar_wait(bar_full + 8 * s, (gi / S) & 1);
                        if (!ok && !fail) fail = 6;
                        front[me] = gi + 1;
                        if (!ok) break;
                        // No proxy fence: the copies' completion reaches the barrier from the copy unit itself
                        // (cp.async.mbarrier.arrive), after the data is in shared memory.
                        asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
                        const unsigned st = ring + s * C::STAGE_BYTES;
                        const int cnt = nt - i < G ? nt - i : G;
                        for (int j = 0; j < cnt; j++)
                        {
                            // gathered rows: MN-major, 128-byte atoms along M two K-atoms apart, K atoms ATOM_BYTES apart
                            const unsigned long long da = make_desc(st + j * C::GB, 2 * C::ATOM_BYTES, C::ATOM_BYTES, (unsigned)C::MODE);
                            // tile values: K-major core matrices (8 rows x 16 B); 16-row tiles keep core (ni, ki) at
                            // (ki*2 + ni)*128, 8-row tiles core (0, ki) at ki*128 - their rows 8-15 of the N = 16 operand
                            // read the unused half of the slot and only feed accumulator columns 8-15, which nobody reads
                            const unsigned a_addr = st + G * C::GB + j * C::A_SLOT;
                            const unsigned long long db = CLS == 1 ? make_desc(a_addr, 256, 128, 0) : make_desc(a_addr, 128, 256, 0);
                            umma<PREC>(tmem_d, da, db, idesc, accumulate);
                            accumulate = 1;
                        }
                        umma_commit(bar_empty + 8 * s);  // frees the slot when these MMAs have read it
                    }
                    if (!ok) break;
                    umma_commit(bar_acc_full + 8 * buf);
                    acc_it++;
                }
                u += stride; cur = nxt;
                nxt = load_unit(u + stride, nunits, nstripes, task_start);
            }
            front[me] = 0x7fffffff;
        }
    }
    else
    {
        // ------------------------------------------------------------ epilogue
        const int quarter = warp & 3;                       // tensor-memory lanes 32*quarter .. +31 belong to this warp
        // M = 128: accumulator row m sits in lane m; M = 64: row m in lane (m/16)*32 + m%16
        const int col = NS == 128 ? quarter * 32 + lane : quarter * 16 + (lane & 15);
        const bool lane_valid = NS == 128 || lane < 16;
        long long u = blockIdx.x;
        Unit cur = load_unit(u, nunits, nstripes, task_start);
        unsigned trow = u < nunits ? __ldg(task_row + cur.task) : 0u;
        int acc_it = 0;
        while (u < nunits && ok)
        {
            const Unit nxt = load_unit(u + stride, nunits, nstripes, task_start);
            const unsigned trow_next = u + stride < nunits ? __ldg(task_row + nxt.task) : 0u;
            const bool split = (trow >> 31) != 0;
            const int first_row = (int)(trow & 0x7fffffffu) - row_begin;
            unsigned r[16];
            if (cur.t1 > cur.t0)
            {
                const int buf = acc_it & 1;
                ok = __all_sync(0xffffffffu, mbar_wait(bar_acc_full + 8 * buf, (acc_it >> 1) & 1));
                if (!ok) fail = 7;
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
                const unsigned taddr = tmem_base + ((unsigned)(quarter * 32) << 16) + (unsigned)(buf * 16);
                if (CLS == 1) tmem_ld16(taddr, r); else tmem_ld8(taddr, r);
                asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
                __syncwarp();
                if (lane == 0) mbar_arrive(bar_acc_empty + 8 * buf);
                acc_it++;
            }
            else
            {
#pragma unroll
                for (int j = 0; j < 16; j++) r[j] = 0u;
            }
            if (lane_valid)
            {
                float *p = dC + (size_t)first_row * (size_t)ldb + (size_t)cur.stripe * NS + col;
#pragma unroll
                for (int n = 0; n < C::BM; n++)
                {
                    if (split) atomicAdd(p + (size_t)n * ldb, __uint_as_float(r[n]));
                    else p[(size_t)n * ldb] = __uint_as_float(r[n]);
                }
            }
            u += stride; cur = nxt; trow = trow_next;
        }
    }
    if (!ok) atomicCAS(err, 0, 0x100 + fail);   // the first failure of the launch is the informative one
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    if (warp == W_MMA)
    {
        asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"(C::TMEM_COLS) : "memory");
    }
}

template <int PREC, int CLS, int NS>
int launch_t(tsp_handle *h, const void *d_b, float *d_c, int colB, cudaStream_t s)
{
    using C = CfgT<PREC, CLS, NS>;
    TspClass &c = h->cls[CLS];
    static int ctas_per_sm[8] = {0};
    auto kern = k_spmm_small_t<PREC, CLS, NS>;
    int &occ = ctas_per_sm[h->device & 7];
    if (occ == 0)
    {
        TSP_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM));
        // CTAs that fit an SM at once, from the kernel's own footprint (the grid is exactly that many per SM)
        cudaFuncAttributes fa;
        TSP_CUDA(cudaFuncGetAttributes(&fa, kern));
        const long long smem_per_cta = C::SMEM + (long long)fa.sharedSizeBytes + 1024;   // + the per-CTA reservation
        const int regs_per_cta = ((fa.numRegs + 7) / 8 * 8) * THREADS;
        long long fit = (long long)h->prop.sharedMemPerMultiprocessor / smem_per_cta;
        if (regs_per_cta > 0 && h->prop.regsPerMultiprocessor / regs_per_cta < fit) fit = h->prop.regsPerMultiprocessor / regs_per_cta;
        if (h->prop.maxThreadsPerMultiProcessor / THREADS < fit) fit = h->prop.maxThreadsPerMultiProcessor / THREADS;
        if (fit > CTAS) fit = CTAS;
        if (fit < 1) { tsp_set_error("transposed small-tile kernel does not fit on an SM"); return TSP_ECUDA; }
        occ = (int)fit;
    }
    const int nstripes = colB / NS;
    const long long units = (long long)c.ntasks * nstripes;
    if (units == 0) return TSP_OK;
    if (units >= (1ll << 31)) { tsp_set_error("transposed small-tile kernel: too many task units"); return TSP_EINVAL; }
    const long long resident = (long long)h->prop.multiProcessorCount * occ;
    const int grid = (int)(units < resident ? units : resident);
    kern<<<grid, THREADS, C::SMEM, s>>>(c.ntasks, nstripes, colB, h->row_begin, c.d_task_row, c.d_task_start, c.d_tile_colidx,
                                        (const unsigned char *)c.d_val, (const unsigned char *)d_b, d_c, h->d_error);
    TSP_CUDA(cudaGetLastError());
    h->launches++;
    return TSP_OK;
}

template <int PREC, int CLS>
int launch_t_width(tsp_handle *h, const void *d_b, float *d_c, int colB, cudaStream_t s)
{
    if (colB % 128 == 0) return launch_t<PREC, CLS, 128>(h, d_b, d_c, colB, s);
    return launch_t<PREC, CLS, 64>(h, d_b, d_c, colB, s);
}

}  // namespace

bool tsp_small_t_supported(int colB) { return colB % 64 == 0; }

int tsp_launch_small_t(tsp_handle *h, int cls, const void *d_b, float *d_c, int colB, cudaStream_t s)
{
    if (!tsp_small_t_supported(colB)) { tsp_set_error("transposed small-tile kernel needs a dense width that is a multiple of 64"); return TSP_EINVAL; }
    if (h->precision == 0)
        return cls == 1 ? launch_t_width<0, 1>(h, d_b, d_c, colB, s) : launch_t_width<0, 2>(h, d_b, d_c, colB, s);
    return cls == 1 ? launch_t_width<1, 1>(h, d_b, d_c, colB, s) : launch_t_width<1, 2>(h, d_b, d_c, colB, s);
}
