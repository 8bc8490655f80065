// Matrix Market (coordinate) reader producing CSR the way the upstream loader does (mmio_allinone,
// src/mmio_highlevel.h:307-480): entries keep FILE ORDER inside each row, repeated entries are kept, symmetric and
// hermitian files are expanded (off-diagonal entries mirrored), pattern files get the value 1.0, integer and
// real values are read as floating point, the imaginary part of complex files is dropped.  Written from scratch
// (one pass over a memory image of the file with strtol/strtod instead of fscanf per line).
#include <ctype.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <string>
#include <vector>

#include "../../include/tilespmm_b200.h"

void tsp_set_error(const char *fmt, ...);

namespace
{
const char *skip_line(const char *p, const char *end)
{
    while (p < end && *p != '\n') p++;
    return p < end ? p + 1 : end;
}
std::string lower(std::string s)
{
    for (char &c : s) c = (char)tolower((unsigned char)c);
    return s;
}
}  // namespace

extern "C" int tsp_read_mtx(const char *path, int *m, int *n, long long *nnz, int *is_symmetric, int **h_rowptr, int **h_colidx,
                            float **h_val)
{
    if (!path || !m || !n || !nnz || !h_rowptr || !h_colidx || !h_val) { tsp_set_error("read_mtx: null argument"); return TSP_EINVAL; }
    FILE *f = fopen(path, "rb");
    if (!f) { tsp_set_error("read_mtx: cannot open %s", path); return TSP_EINVAL; }
    fseek(f, 0, SEEK_END);
    const long size = ftell(f);
    fseek(f, 0, SEEK_SET);
    std::vector<char> buf((size_t)size + 1);
    if (size > 0 && fread(buf.data(), 1, (size_t)size, f) != (size_t)size) { fclose(f); tsp_set_error("read_mtx: short read"); return TSP_EINVAL; }
    fclose(f);
    buf[(size_t)size] = 0;
    const char *p = buf.data(), *end = p + size;

    // banner: %%MatrixMarket matrix coordinate <field> <symmetry>   (two percent signs, src/mmio.h:19)
    char b0[64] = "", b1[64] = "", b2[64] = "", b3[64] = "", b4[64] = "";
    if (sscanf(p, "%63s %63s %63s %63s %63s", b0, b1, b2, b3, b4) != 5 || strncmp(b0, "%%MatrixMarket", 14) != 0)
    {
        tsp_set_error("read_mtx: could not process the Matrix Market banner of %s", path);
        return TSP_EINVAL;
    }
    const std::string object = lower(b1), format = lower(b2), field = lower(b3), symm = lower(b4);
    if (object != "matrix" || format != "coordinate")
    {
        tsp_set_error("read_mtx: only 'matrix coordinate' files are supported (%s %s)", b1, b2);
        return TSP_EINVAL;
    }
    const bool pattern = field == "pattern", cplx = field == "complex";
    if (!pattern && !cplx && field != "real" && field != "integer" && field != "double")
    {
        tsp_set_error("read_mtx: unknown field '%s'", b3);
        return TSP_EINVAL;
    }
    const bool mirrored = symm == "symmetric" || symm == "hermitian";
    p = skip_line(p, end);
    while (p < end && (*p == '%' || *p == '\n' || *p == '\r')) p = skip_line(p, end);
    char *q = nullptr;
    const long rows = strtol(p, &q, 10); p = q;
    const long cols = strtol(p, &q, 10); p = q;
    const long long entries = strtoll(p, &q, 10); p = q;
    if (rows <= 0 || cols <= 0 || entries < 0 || rows > 0x7fffffffL || cols > 0x7fffffffL)
    {
        tsp_set_error("read_mtx: bad size line in %s", path);
        return TSP_EINVAL;
    }
    std::vector<int> ri((size_t)entries), ci((size_t)entries);
    std::vector<float> va((size_t)entries);
    std::vector<long long> count((size_t)rows + 1, 0);
    for (long long e = 0; e < entries; e++)
    {
        const long i = strtol(p, &q, 10);
        if (q == p) { tsp_set_error("read_mtx: %s ends after %lld of %lld entries", path, e, entries); return TSP_EINVAL; }
        p = q;
        const long j = strtol(p, &q, 10); p = q;
        double v = 1.0;
        if (!pattern) { v = strtod(p, &q); p = q; if (cplx) { (void)strtod(p, &q); p = q; } }
        if (i < 1 || i > rows || j < 1 || j > cols) { tsp_set_error("read_mtx: entry %lld of %s is out of range", e + 1, path); return TSP_EINVAL; }
        ri[(size_t)e] = (int)(i - 1); ci[(size_t)e] = (int)(j - 1); va[(size_t)e] = (float)v;
        count[(size_t)i - 1]++;
        if (mirrored && i != j)
        {
            if (j > rows) { tsp_set_error("read_mtx: symmetric file %s is not square", path); return TSP_EINVAL; }
            count[(size_t)j - 1]++;
        }
    }
    long long total = 0;
    for (long r = 0; r <= rows; r++) { const long long c = r < rows ? count[(size_t)r] : 0; count[(size_t)r] = total; total += c; }
    if (total > 0x7fffffffLL) { tsp_set_error("read_mtx: %lld stored entries exceed 32-bit indices", total); return TSP_EINVAL; }
    int *rp = (int *)malloc(((size_t)rows + 1) * sizeof(int));
    int *cx = (int *)malloc((size_t)(total ? total : 1) * sizeof(int));
    float *vx = (float *)malloc((size_t)(total ? total : 1) * sizeof(float));
    if (!rp || !cx || !vx) { free(rp); free(cx); free(vx); tsp_set_error("read_mtx: out of host memory"); return TSP_ENOMEM; }
    for (long r = 0; r <= rows; r++) rp[r] = (int)count[(size_t)r];
    std::vector<long long> fill(count.begin(), count.end() - 1);
    for (long long e = 0; e < entries; e++)  // file order, the mirrored copy right after its original
    {
        const int i = ri[(size_t)e], j = ci[(size_t)e];
        long long o = fill[(size_t)i]++;
        cx[o] = j; vx[o] = va[(size_t)e];
        if (mirrored && i != j) { o = fill[(size_t)j]++; cx[o] = i; vx[o] = va[(size_t)e]; }
    }
    *m = (int)rows; *n = (int)cols; *nnz = total;
    if (is_symmetric) *is_symmetric = mirrored ? 1 : 0;
    *h_rowptr = rp; *h_colidx = cx; *h_val = vx;
    return TSP_OK;
}

extern "C" void tsp_free_host(void *p) { free(p); }
