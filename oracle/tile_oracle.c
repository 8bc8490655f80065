/* TEST INFRASTRUCTURE ONLY -- never linked into, imported by or executed from the product library.
 *
 * Plain-C restatement (CPU) of the upstream TileSpMM hot path, used as the checker in tests, in the
 * smoke entry and as the timed CPU baseline:
 *   - orc_split      : gamma/delta greedy row partitioner          (upstream src/hetero_split.h:144-291)
 *   - orc_convert    : CSR -> column-compacted tiles per class     (upstream src/csr2tile.h:15-379, 724-795)
 *   - orc_top4       : threshold cost model, four cheapest TH      (upstream src/csr2tile.h:437-642)
 *   - orc_schedule   : panel -> task splitting for one TH          (upstream src/csr2tile.h:383-434)
 *   - orc_spmm_csr   : CSR SpMM, FP32 accumulation in CSR order    (the upstream check compares against
 *                      cuSPARSE, src/main.cu:315-335; upstream has no CPU SpMM, so this is the numerical
 *                      oracle and the CPU baseline)
 * Parity of this file is pinned against the upstream sources themselves, compiled unmodified into
 * oracle/_ref/libref_{fp16,tf32}.so (see ref_driver.cu), on seeded inputs, and against the golden
 * digests committed under tests/golden/ that were produced by those upstream objects.
 *
 * Values: precision 0 = FP16 (bit patterns in uint16_t), precision 1 = TF32 (plain float).
 * Classes: 0 = 64-row panels, 1 = 16-row panels, 2 = 8-row panels.
 */
#include <math.h>
#include <omp.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

typedef struct
{
    int precision;          /* 0 fp16, 1 tf32 */
    int rowA, colA;
    int BM[3], BN[3];
    int rows[3];            /* rows assigned to each class */
    long long nnz[3];
    int *orig_row[3];       /* original row of every class row, in class order */
    int tilem[3], tilenum[3];
    int *tile_ptr[3];       /* tilem+1 */
    int *tile_nnz[3];       /* tilenum+1 */
    int *tile_colidx[3];    /* tilenum*BN */
    void *tile_val[3];      /* tilenum*BM*BN values, upstream fragment order */
    int *panel_row[3];      /* tilem: original first row of each panel */
} OrcTiles;

/* ---------------------------------------------------------------- distinct column counting */

typedef struct { int *stamp; int tick; } Marker;

static int distinct_cols(Marker *mk, const int *rowptr, const int *colidx, int r0, int r1)
{
    int n = 0;
    mk->tick++;
    for (int j = rowptr[r0]; j < rowptr[r1]; j++)
        if (mk->stamp[colidx[j]] != mk->tick) { mk->stamp[colidx[j]] = mk->tick; n++; }
    return n;
}

/* Upstream src/hetero_split.h:144-291.  Writes cls_of_start: for every panel, in scan order, its first
 * row and class.  Returns the number of panels. */
static int split_scan(int rowA, int colA, const int *rowptr, const int *colidx, float gamma, float delta,
                      int *panel_start, int *panel_cls)
{
    int np = 0;
    /* shortcuts (hetero_split.h:152-169) */
    int fixed = -1;
    if (gamma <= 0.0f) fixed = 0;
    else if (gamma >= 4.0f && delta <= 0.0f) fixed = 1;
    else if (gamma >= 4.0f && delta > 2.0f) fixed = 2;
    if (fixed >= 0)
    {
        int step = fixed == 0 ? 64 : (fixed == 1 ? 16 : 8);
        for (int i = 0; i < rowA; i += step) { panel_start[np] = i; panel_cls[np] = fixed; np++; }
        return np;
    }
    Marker mk;
    mk.stamp = (int *)calloc((size_t)(colA > 0 ? colA : 1), sizeof(int));
    mk.tick = 0;
    int i = 0;
    while (i < rowA)
    {
        int is64 = 0, n16_first = -1;
        if (gamma < 4.0f && i + 64 <= rowA) /* hetero_split.h:204-229 */
        {
            int n64 = distinct_cols(&mk, rowptr, colidx, i, i + 64);
            if (n64 > 0)
            {
                float thr = gamma * n64;
                int s16 = 0;
                for (int q = 0; q < 4 && !is64; q++)
                {
                    int n16 = distinct_cols(&mk, rowptr, colidx, i + 16 * q, i + 16 * q + 16);
                    if (q == 0) n16_first = n16;
                    s16 += n16;
                    if (s16 > thr) is64 = 1;
                }
            }
        }
        if (is64) { panel_start[np] = i; panel_cls[np] = 0; np++; i += 64; continue; }

        int is16 = 0;
        if (delta <= 0.0f) is16 = 1; /* hetero_split.h:242-244: also for the ragged tail */
        else if (!(delta > 2.0f) && i + 16 <= rowA) /* hetero_split.h:245-260 */
        {
            int n16 = n16_first >= 0 ? n16_first : distinct_cols(&mk, rowptr, colidx, i, i + 16);
            if (n16 > 0)
            {
                float thr = delta * n16;
                int s8 = distinct_cols(&mk, rowptr, colidx, i, i + 8);
                if (s8 >= thr) is16 = 1;
                else
                {
                    s8 += distinct_cols(&mk, rowptr, colidx, i + 8, i + 16);
                    if (s8 >= thr) is16 = 1;
                }
            }
        }
        if (is16) { panel_start[np] = i; panel_cls[np] = 1; np++; i += 16; continue; }
        panel_start[np] = i; panel_cls[np] = 2; np++; i += 8;
    }
    free(mk.stamp);
    return np;
}

/* ---------------------------------------------------------------- fragment permutations */

/* Position of element (r,c) of a 16 x KW block in the upstream A-fragment order
 * (src/csr2tile.h:289-307): KW = 16 for FP16, 8 for TF32. */
static inline int frag16_index(int precision, int r, int c)
{
    if (precision == 0)
    {
        int lane = ((r & 7) << 2) + ((c & 7) >> 1);
        int slot = ((c >> 3) << 2) + ((r >> 3) << 1) + (c & 1);
        return lane * 8 + slot;
    }
    int lane = ((r & 7) << 2) + (c & 3);
    int slot = ((c >> 2) << 1) + (r >> 3);
    return lane * 4 + slot;
}

/* Position of element (r,c) inside one tile of class BM (src/csr2tile.h:255-373). */
static inline int tile_index(int precision, int BM, int BN, int r, int c)
{
    if (BM == 8) /* src/csr2tile.h:262-271: the tile is the k x n8 operand */
    {
        if (precision == 0) return (((r << 2) + ((c >> 1) & 3)) << 2) + ((c >> 3) << 1) + (c & 1);
        return (((r << 2) + (c & 3)) << 1) + (c >> 2);
    }
    int KW = precision == 0 ? 16 : 8;
    if (BM == 16) return frag16_index(precision, r, c);
    int nsubk = BN / KW; /* BM == 64: 4 x nsubk sub-blocks, sub_m-major (src/csr2tile.h:319-372) */
    int sub = (r >> 4) * nsubk + c / KW;
    return sub * 16 * KW + frag16_index(precision, r & 15, c % KW);
}

/* ---------------------------------------------------------------- conversion */

static int cmp_int(const void *a, const void *b)
{
    int x = *(const int *)a, y = *(const int *)b;
    return (x > y) - (x < y);
}

static void scan_exclusive(int *a, int n)
{
    int run = 0;
    for (int i = 0; i < n; i++) { int v = a[i]; a[i] = run; run += v; }
}

/* Upstream Tile_create (src/csr2tile.h:724-795) for one class whose rows are orig_row[0..rows). */
static void convert_class(OrcTiles *T, int cls, const int *rowptr, const int *colidx, const void *val)
{
    const int BM = T->BM[cls], BN = T->BN[cls], rows = T->rows[cls], prec = T->precision;
    const int *orow = T->orig_row[cls];
    const int tilem = (rows + BM - 1) / BM;
    T->tilem[cls] = tilem;
    T->tile_ptr[cls] = (int *)calloc((size_t)tilem + 1, sizeof(int));
    T->panel_row[cls] = (int *)malloc(sizeof(int) * (size_t)(tilem > 0 ? tilem : 1));
    for (int p = 0; p < tilem; p++) T->panel_row[cls][p] = orow[p * BM];

    const int colA = T->colA;
    int nth = omp_get_max_threads();
    int *stamp_g = (int *)calloc((size_t)nth * colA, sizeof(int));
    int *rank_g = (int *)malloc(sizeof(int) * (size_t)nth * colA);
    int *list_g = (int *)malloc(sizeof(int) * (size_t)nth * colA);

    /* pass 1: tiles per panel = ceil(distinct/BN) (src/csr2tile.h:15-56) */
#pragma omp parallel for schedule(dynamic, 32)
    for (int p = 0; p < tilem; p++)
    {
        int *stamp = stamp_g + (size_t)omp_get_thread_num() * colA;
        int r1 = p * BM + BM < rows ? p * BM + BM : rows, n = 0;
        for (int r = p * BM; r < r1; r++)
            for (int j = rowptr[orow[r]]; j < rowptr[orow[r] + 1]; j++)
                if (stamp[colidx[j]] != p + 1) { stamp[colidx[j]] = p + 1; n++; }
        T->tile_ptr[cls][p] = (n + BN - 1) / BN;
    }
    scan_exclusive(T->tile_ptr[cls], tilem + 1);
    const int tilenum = T->tile_ptr[cls][tilem];
    T->tilenum[cls] = tilenum;
    T->tile_nnz[cls] = (int *)calloc((size_t)tilenum + 1, sizeof(int));
    T->tile_colidx[cls] = (int *)malloc(sizeof(int) * (size_t)(tilenum > 0 ? tilenum : 1) * BN);
    size_t vsz = prec == 0 ? 2 : 4;
    T->tile_val[cls] = calloc((size_t)(tilenum > 0 ? tilenum : 1) * BM * BN, vsz);
    memset(stamp_g, 0, sizeof(int) * (size_t)nth * colA);

    /* pass 2: sorted distinct columns, padding, per-tile nnz, values (src/csr2tile.h:61-379) */
#pragma omp parallel for schedule(dynamic, 32)
    for (int p = 0; p < tilem; p++)
    {
        int tid = omp_get_thread_num();
        int *stamp = stamp_g + (size_t)tid * colA, *rank = rank_g + (size_t)tid * colA,
            *list = list_g + (size_t)tid * colA;
        int t0 = T->tile_ptr[cls][p], nt = T->tile_ptr[cls][p + 1] - t0;
        if (nt == 0) continue;
        int r1 = p * BM + BM < rows ? p * BM + BM : rows, n = 0;
        for (int r = p * BM; r < r1; r++)
            for (int j = rowptr[orow[r]]; j < rowptr[orow[r] + 1]; j++)
                if (stamp[colidx[j]] != p + 1) { stamp[colidx[j]] = p + 1; list[n++] = colidx[j]; }
        qsort(list, (size_t)n, sizeof(int), cmp_int);
        for (int k = 0; k < n; k++) { rank[list[k]] = k; T->tile_colidx[cls][(size_t)t0 * BN + k] = list[k]; }
        for (int k = n; k < nt * BN; k++) T->tile_colidx[cls][(size_t)t0 * BN + k] = list[n - 1];
        for (int r = p * BM; r < r1; r++)
        {
            int ri = r - p * BM;
            for (int j = rowptr[orow[r]]; j < rowptr[orow[r] + 1]; j++)
            {
                int k = rank[colidx[j]], t = k / BN, c = k % BN;
                T->tile_nnz[cls][t0 + t]++;
                size_t pos = (size_t)(t0 + t) * BM * BN + tile_index(prec, BM, BN, ri, c);
                if (prec == 0) /* duplicates are summed in value type, CSR order (src/csr2tile.h:271,283,318) */
                {
                    _Float16 *dst = (_Float16 *)T->tile_val[cls] + pos;
                    _Float16 v;
                    memcpy(&v, (const uint16_t *)val + j, 2);
                    *dst = (_Float16)((float)*dst + (float)v);
                }
                else
                {
                    float *dst = (float *)T->tile_val[cls] + pos;
                    *dst += ((const float *)val)[j];
                }
            }
        }
    }
    scan_exclusive(T->tile_nnz[cls], tilenum + 1);
    free(stamp_g); free(rank_g); free(list_g);
}

/* matrix_split + three Tile_create calls, as in upstream src/main.cu:251-276. */
OrcTiles *orc_convert(int precision, int rowA, int colA, const int *rowptr, const int *colidx, const void *val,
                      float gamma, float delta)
{
    OrcTiles *T = (OrcTiles *)calloc(1, sizeof(OrcTiles));
    T->precision = precision; T->rowA = rowA; T->colA = colA;
    T->BM[0] = 64; T->BM[1] = 16; T->BM[2] = 8;
    T->BN[0] = precision ? 16 : 32; T->BN[1] = precision ? 8 : 16; T->BN[2] = precision ? 8 : 16;
    int maxp = rowA / 8 + 2;
    int *pstart = (int *)malloc(sizeof(int) * maxp), *pcls = (int *)malloc(sizeof(int) * maxp);
    int np = split_scan(rowA, colA, rowptr, colidx, gamma, delta, pstart, pcls);
    for (int c = 0; c < 3; c++) T->orig_row[c] = (int *)malloc(sizeof(int) * (size_t)(rowA > 0 ? rowA : 1));
    for (int p = 0; p < np; p++)
    {
        int c = pcls[p], end = pstart[p] + T->BM[c] < rowA ? pstart[p] + T->BM[c] : rowA;
        for (int r = pstart[p]; r < end; r++)
        {
            T->orig_row[c][T->rows[c]++] = r;
            T->nnz[c] += rowptr[r + 1] - rowptr[r];
        }
    }
    free(pstart); free(pcls);
    for (int c = 0; c < 3; c++)
        if (T->rows[c] > 0) convert_class(T, c, rowptr, colidx, val); /* src/main.cu:266-275 */
    return T;
}

void orc_info(const OrcTiles *T, int *info12)
{
    for (int c = 0; c < 3; c++)
    {
        info12[c * 4 + 0] = T->rows[c];
        info12[c * 4 + 1] = (int)T->nnz[c];
        info12[c * 4 + 2] = T->tilem[c];
        info12[c * 4 + 3] = T->tilenum[c];
    }
}

/* which: 0 orig_row, 1 tile_ptr, 2 tile_nnz, 3 tile_colidx, 4 tile values, 5 panel first rows */
long long orc_array(const OrcTiles *T, int cls, int which, void *dst)
{
    const void *src = NULL;
    size_t bytes = 0;
    if (T->rows[cls] == 0) return 0;
    switch (which)
    {
    case 0: src = T->orig_row[cls]; bytes = (size_t)T->rows[cls] * 4; break;
    case 1: src = T->tile_ptr[cls]; bytes = ((size_t)T->tilem[cls] + 1) * 4; break;
    case 2: src = T->tile_nnz[cls]; bytes = ((size_t)T->tilenum[cls] + 1) * 4; break;
    case 3: src = T->tile_colidx[cls]; bytes = (size_t)T->tilenum[cls] * T->BN[cls] * 4; break;
    case 4: src = T->tile_val[cls];
            bytes = (size_t)T->tilenum[cls] * T->BM[cls] * T->BN[cls] * (T->precision ? 4 : 2); break;
    case 5: src = T->panel_row[cls]; bytes = (size_t)T->tilem[cls] * 4; break;
    default: return -1;
    }
    if (dst && bytes) memcpy(dst, src, bytes);
    return (long long)bytes;
}

void orc_destroy(OrcTiles *T)
{
    if (!T) return;
    for (int c = 0; c < 3; c++)
    {
        free(T->orig_row[c]); free(T->tile_ptr[c]); free(T->tile_nnz[c]);
        free(T->tile_colidx[c]); free(T->tile_val[c]); free(T->panel_row[c]);
    }
    free(T);
}

/* ---------------------------------------------------------------- scheduling */

/* Upstream tile_pretreatment (src/csr2tile.h:383-434).  rows/colstart may be NULL (count only). */
int orc_schedule(const OrcTiles *T, int cls, int TH, unsigned int *rows, int *colstart)
{
    if (T->tilenum[cls] == 0) return 0;
    const int *tp = T->tile_ptr[cls];
    int ntask = 0;
    if (colstart) colstart[0] = tp[0];
    for (int p = 0; p < T->tilem[cls]; p++)
    {
        int len = tp[p + 1] - tp[p];
        if (len <= TH)
        {
            if (rows) rows[ntask] = (unsigned int)T->panel_row[cls][p];
            if (colstart) colstart[ntask + 1] = tp[p + 1];
            ntask++;
        }
        else
        {
            int parts = (int)ceil((double)len / (double)TH);
            int each = (int)ceil((double)len / (double)parts);
            for (int s = 0; s < parts; s++)
            {
                if (rows) rows[ntask] = (unsigned int)T->panel_row[cls][p] | 0x80000000u;
                if (colstart) colstart[ntask + 1] = s == parts - 1 ? tp[p + 1] : tp[p] + (s + 1) * each;
                ntask++;
            }
        }
    }
    return ntask;
}

/* Device limits and the resources of the kernel that serves (class, colB) -- what the upstream
 * platform probe records (pre/prefetch_probe.cu:12-28, 62-95). */
typedef struct
{
    int sm_count, threads_per_sm, blocks_per_sm, registers_per_sm, l2_bytes;
    long long shared_bytes_per_sm;
    int threads, registers_per_thread, iteration_bytes;
    long long shared_bytes;
    /* launch geometry of the kernel: tasks served by one block and column stripes per task.  Upstream:
     * 4 tasks per block for the 32-column 8/16-row kernels, else 1; ceil(colB/64) stripes, 1 when colB == 32
     * (src/csr2tile.h:590-601). */
    int tasks_per_block, stripes;
    /* weight of one atomic slice.  Upstream hard-codes a table "calibrated from existing platform data"
     * (src/csr2tile.h:483-495); 0 selects that table, any other value stands in for a platform's own calibration. */
    float atom_weight;
} OrcResources;

/* Upstream get_optimal_prefetch_th (src/csr2tile.h:437-642); float arithmetic in upstream's order. */
int orc_top4(const OrcTiles *T, int cls, int colB, const OrcResources *R, int *top4)
{
    const int BM = T->BM[cls], is_tf32 = T->precision, tilem = T->tilem[cls];
    const int *tp = T->tile_ptr[cls];
    for (int i = 0; i < 4; i++) top4[i] = 32;
    if (T->tilenum[cls] == 0) return 0;

    int blk_reg = R->registers_per_sm / (R->registers_per_thread * R->threads);
    int blk_smem = R->shared_bytes > 0 ? (int)(R->shared_bytes_per_sm / R->shared_bytes) : R->blocks_per_sm;
    int blk_sm = R->threads_per_sm / R->threads;
    if (blk_reg < blk_sm) blk_sm = blk_reg;
    if (blk_smem < blk_sm) blk_sm = blk_smem;
    if (blk_sm > R->blocks_per_sm) blk_sm = R->blocks_per_sm;
    if (blk_sm <= 0) return 1;
    float cap = (float)(blk_sm * R->sm_count);
    float lambda_l2 = (float)(R->iteration_bytes * cap) / (float)R->l2_bytes;
    float lambda_atom = 0.01f; /* table at src/csr2tile.h:484-495 */
    if (colB == 32)
    {
        if (BM == 64) lambda_atom = is_tf32 ? 0.020f : 0.019f;
        else if (BM == 16) lambda_atom = is_tf32 ? 0.00830f : 0.00844f;
        else lambda_atom = is_tf32 ? 0.00674f : 0.00360f;
    }
    else
    {
        if (BM == 16) lambda_atom = is_tf32 ? 0.01048f : 0.01163f;
        else if (BM == 8) lambda_atom = is_tf32 ? 0.00960f : 0.00826f;
    }
    if (R->atom_weight != 0.0f) lambda_atom = R->atom_weight;
    float atom_per_col = lambda_atom * (1.0f / 32.0f);

    int max_len = 0;
    long long total_len = 0;
    for (int p = 0; p < tilem; p++)
    {
        int len = tp[p + 1] - tp[p];
        if (len > max_len) max_len = len;
        total_len += len;
    }
    if (max_len == 0) return 0;
    int *hist = (int *)calloc((size_t)max_len + 1, sizeof(int));
    for (int p = 0; p < tilem; p++) hist[tp[p + 1] - tp[p]]++;
    hist[0] = 0;

    float avg_len = (float)total_len / tilem;
    float atom_pen = atom_per_col * (float)colB;
    if (max_len > avg_len * 5.0f) atom_pen *= 0.04f; /* src/csr2tile.h:549 */
    int tmax = (max_len + 7) / 8 * 8;
    if (tmax > 128) tmax = 128;

    int cand_th[16];
    float cand_cost[16];
    int ncand = 0;
    long long prev_tasks = -1;
    for (int TH = 8; TH <= tmax; TH += 8)
    {
        long long atom_ops = 0, tasks = 0;
        int max_chunk = 0;
        float l2_penalty = 0.0f;
        for (int len = 1; len <= max_len; len++)
        {
            int cnt = hist[len];
            if (!cnt) continue;
            int parts = (len + TH - 1) / TH, each = (len + parts - 1) / parts;
            atom_ops += (long long)(parts - 1) * cnt;
            tasks += (long long)parts * cnt;
            if (each > max_chunk) max_chunk = each;
            if (parts > 1) l2_penalty += (1.0f - (1.0f / (float)parts)) * cnt;
        }
        if (tasks == prev_tasks) continue; /* src/csr2tile.h:586-588 */
        prev_tasks = tasks;
        long long blocks = (tasks * R->stripes + R->tasks_per_block - 1) / R->tasks_per_block;
        float cost_base = (float)blocks / cap * TH;
        float cost_tail = (float)max_chunk;
        float cost_l2 = l2_penalty * lambda_l2;
        float cost_comp = cost_base + cost_tail + cost_l2; /* src/csr2tile.h:603-612 */
        float cost_atom = atom_pen * atom_ops;
        cand_th[ncand] = TH;
        cand_cost[ncand] = cost_comp + cost_atom;
        ncand++;
    }
    /* stable ascending order: an insertion sort that only moves on strict '>' keeps ties in TH order,
     * like the bubble sort at src/csr2tile.h:620-631 */
    for (int i = 1; i < ncand; i++)
    {
        int th = cand_th[i]; float c = cand_cost[i]; int j = i - 1;
        while (j >= 0 && cand_cost[j] > c) { cand_th[j + 1] = cand_th[j]; cand_cost[j + 1] = cand_cost[j]; j--; }
        cand_th[j + 1] = th; cand_cost[j + 1] = c;
    }
    for (int i = 0; i < 4; i++) top4[i] = i < ncand ? cand_th[i] : cand_th[0];
    free(hist);
    return 0;
}

/* ---------------------------------------------------------------- CPU CSR SpMM (numerical oracle + CPU baseline) */

static inline float half_bits_to_float(uint16_t h)
{
    _Float16 v;
    memcpy(&v, &h, 2);
    return (float)v;
}

static inline float tf32_trunc(float x) /* the tensor core ignores the low 13 mantissa bits */
{
    uint32_t u;
    memcpy(&u, &x, 4);
    u &= 0xFFFFE000u;
    memcpy(&x, &u, 4);
    return x;
}

/* C[rowA x ldc] = A * B, FP32 accumulate in CSR order; rows [row0,row1).  B is colA x ldb.
 * precision 0: A, B are FP16 bit patterns; precision 1: floats, truncated to TF32 when trunc != 0. */
void orc_spmm_csr(int precision, int trunc, int row0, int row1, const int *rowptr, const int *colidx,
                  const void *val, const void *B, int ldb, int ncols, float *C, int ldc)
{
#pragma omp parallel for schedule(dynamic, 64)
    for (int r = row0; r < row1; r++)
    {
        float *c = C + (size_t)r * ldc;
        for (int n = 0; n < ncols; n++) c[n] = 0.0f;
        for (int j = rowptr[r]; j < rowptr[r + 1]; j++)
        {
            if (precision == 0)
            {
                float a = half_bits_to_float(((const uint16_t *)val)[j]);
                const uint16_t *b = (const uint16_t *)B + (size_t)colidx[j] * ldb;
                for (int n = 0; n < ncols; n++) c[n] += a * half_bits_to_float(b[n]);
            }
            else
            {
                float a = ((const float *)val)[j];
                const float *b = (const float *)B + (size_t)colidx[j] * ldb;
                if (trunc)
                {
                    a = tf32_trunc(a);
                    for (int n = 0; n < ncols; n++) c[n] += a * tf32_trunc(b[n]);
                }
                else
                    for (int n = 0; n < ncols; n++) c[n] += a * b[n];
            }
        }
    }
}

int orc_num_threads(void) { return omp_get_max_threads(); }

/* Launchers such as torchrun export OMP_NUM_THREADS=1; the CPU baseline is meant to use every host core. */
void orc_set_threads(int n) { if (n > 0) omp_set_num_threads(n); }
