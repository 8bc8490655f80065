// Tile cache on disk: the converted matrix of a handle (all three classes, device layout) written to and read
// back from one binary file, so that a large conversion is done once per matrix and (gamma, delta).  Upstream has no
// counterpart (it converts on every run); the file is private to this library (magic + version checked on load).
#include <stdio.h>
#include <string.h>

#include <vector>

#include "tsp_internal.cuh"

namespace
{
const char kMagic[8] = {'T', 'S', 'P', 'T', 'I', 'L', 'E', '2'};

struct FileHeader
{
    char magic[8];
    int version, precision, rowA, colA;
    long long nnzA;
    int row_begin, row_end;
    int rows[3], tilem[3], tilenum[3];
    long long nnz[3];
    long long pack_bytes;   // records of the 64-row class
};

int write_dev(FILE *f, const void *d, size_t bytes, std::vector<unsigned char> &tmp)
{
    if (bytes == 0) return TSP_OK;
    tmp.resize(bytes);
    TSP_CUDA(cudaMemcpy(tmp.data(), d, bytes, cudaMemcpyDeviceToHost));
    if (fwrite(tmp.data(), 1, bytes, f) != bytes) { tsp_set_error("save: short write"); return TSP_EINVAL; }
    return TSP_OK;
}

// reads `bytes` from the file into host memory (kept in tmp for checking) and copies them to the device
int read_dev(FILE *f, void *d, size_t bytes, std::vector<unsigned char> &tmp)
{
    tmp.resize(bytes);
    if (bytes == 0) return TSP_OK;
    if (fread(tmp.data(), 1, bytes, f) != bytes) { tsp_set_error("load: file is truncated"); return TSP_EINVAL; }
    TSP_CUDA(cudaMemcpy(d, tmp.data(), bytes, cudaMemcpyHostToDevice));
    return TSP_OK;
}

int bad_file(const char *what)
{
    tsp_set_error("load: the file is inconsistent (%s); refusing to use it", what);
    return TSP_EINVAL;
}
}  // namespace

extern "C" int tsp_save(const tsp_handle *h, const char *path)
{
    if (!h || !path) { tsp_set_error("save: null argument"); return TSP_EINVAL; }
    if (!h->converted) { tsp_set_error("save: convert first"); return TSP_ESTATE; }
    TSP_CUDA(cudaSetDevice(h->device));
    FILE *f = fopen(path, "wb");
    if (!f) { tsp_set_error("save: cannot open %s", path); return TSP_EINVAL; }
    FileHeader hd;
    memset(&hd, 0, sizeof(hd));
    memcpy(hd.magic, kMagic, 8);
    hd.version = 2; hd.precision = h->precision; hd.rowA = h->rowA; hd.colA = h->colA; hd.nnzA = h->nnzA;
    hd.row_begin = h->row_begin; hd.row_end = h->row_end; hd.pack_bytes = h->cls[0].pack_bytes;
    for (int k = 0; k < 3; k++) { hd.rows[k] = h->cls[k].rows; hd.tilem[k] = h->cls[k].tilem; hd.tilenum[k] = h->cls[k].tilenum; hd.nnz[k] = h->cls[k].nnz; }
    int rc = fwrite(&hd, sizeof(hd), 1, f) == 1 ? TSP_OK : TSP_EINVAL;
    std::vector<unsigned char> tmp;
    const size_t vsz = h->precision ? 4 : 2;
    for (int k = 0; k < 3 && rc == TSP_OK; k++)
    {
        const TspClass &c = h->cls[k];
        if (fwrite(c.h_tile_ptr.data(), 4, (size_t)c.tilem + 1, f) != (size_t)c.tilem + 1) rc = TSP_EINVAL;
        if (rc == TSP_OK && c.tilem && fwrite(c.h_panel_row.data(), 4, (size_t)c.tilem, f) != (size_t)c.tilem) rc = TSP_EINVAL;
        if (rc == TSP_OK) rc = write_dev(f, c.d_tile_nnz, ((size_t)c.tilenum + 1) * 4, tmp);
        if (rc == TSP_OK) rc = write_dev(f, c.d_tile_colidx, (size_t)c.tilenum * c.BN * 4, tmp);
        if (k == 0)
        {
            if (rc == TSP_OK) rc = write_dev(f, c.d_bitmap, (size_t)c.tilenum * tsp_mask_bytes(h->precision), tmp);
            if (rc == TSP_OK) rc = write_dev(f, c.d_rec, ((size_t)c.tilenum + 1) * 4, tmp);
            if (rc == TSP_OK) rc = write_dev(f, c.d_pack, (size_t)c.pack_bytes, tmp);
        }
        else if (rc == TSP_OK) rc = write_dev(f, c.d_val, (size_t)c.tilenum * c.BM * c.BN * vsz, tmp);
    }
    if (fclose(f) != 0 && rc == TSP_OK) rc = TSP_EINVAL;
    if (rc == TSP_EINVAL) tsp_set_error("save: writing %s failed", path);
    return rc;
}

// Everything the kernels later use as an index is checked here, on the host, before it reaches the device: a damaged or
// stale file must come back as an error, not as an out-of-bounds access on the GPU.
extern "C" int tsp_load(tsp_handle *h, const char *path)
{
    if (!h || !path) { tsp_set_error("load: null argument"); return TSP_EINVAL; }
    TSP_CUDA(cudaSetDevice(h->device));
    FILE *f = fopen(path, "rb");
    if (!f) { tsp_set_error("load: cannot open %s", path); return TSP_EINVAL; }
    FileHeader hd;
    if (fread(&hd, sizeof(hd), 1, f) != 1 || memcmp(hd.magic, kMagic, 8) != 0 || hd.version != 2)
    {
        fclose(f);
        tsp_set_error("load: %s is not a tile cache of this version of the library", path);
        return TSP_EINVAL;
    }
    if (hd.precision != h->precision)
    {
        fclose(f);
        tsp_set_error("load: %s holds %s tiles but the handle was created for %s", path, hd.precision ? "TF32" : "FP16", h->precision ? "TF32" : "FP16");
        return TSP_EINVAL;
    }
    // header fields: shapes, shard rows, counts (bounded by what a conversion can produce)
    bool ok = hd.rowA > 0 && hd.colA > 0 && hd.nnzA >= 0 && hd.nnzA <= 0x7fffffffLL && hd.row_begin >= 0 && hd.row_begin <= hd.row_end &&
              hd.row_end <= hd.rowA && hd.pack_bytes >= 0 && hd.pack_bytes % 16 == 0 && hd.pack_bytes < (0x7fffffffLL << 4);
    for (int k = 0; k < 3 && ok; k++)
        ok = hd.tilem[k] >= 0 && hd.tilem[k] <= hd.rowA / 8 + 1 && hd.tilenum[k] >= 0 && (long long)hd.tilenum[k] <= hd.nnzA && hd.rows[k] >= 0 &&
             hd.rows[k] <= hd.rowA && hd.nnz[k] >= 0 && hd.nnz[k] <= hd.nnzA;
    if (!ok) { fclose(f); return bad_file("header"); }
    tsp_free_tiles(h);
    h->rowA = hd.rowA; h->colA = hd.colA; h->nnzA = hd.nnzA; h->row_begin = hd.row_begin; h->row_end = hd.row_end;
    for (int k = 0; k < 3; k++) { TspClass &c = h->cls[k]; c.rows = hd.rows[k]; c.tilem = hd.tilem[k]; c.tilenum = hd.tilenum[k]; c.nnz = hd.nnz[k]; }
    std::vector<unsigned char> tmp;
    const size_t vsz = h->precision ? 4 : 2;
    int rc = tsp_alloc_tile_arrays(h);
    if (rc == TSP_OK && hd.pack_bytes > 0) rc = tsp_alloc_pack(h, hd.pack_bytes);
    for (int k = 0; k < 3 && rc == TSP_OK; k++)
    {
        TspClass &c = h->cls[k];
        try { c.h_tile_ptr.resize((size_t)c.tilem + 1); c.h_panel_row.resize(c.tilem); }
        catch (...) { tsp_set_error("load: out of host memory"); rc = TSP_ENOMEM; break; }
        if (fread(c.h_tile_ptr.data(), 4, (size_t)c.tilem + 1, f) != (size_t)c.tilem + 1) rc = TSP_EINVAL;
        if (rc == TSP_OK && c.tilem && fread(c.h_panel_row.data(), 4, (size_t)c.tilem, f) != (size_t)c.tilem) rc = TSP_EINVAL;
        if (rc == TSP_EINVAL) { tsp_set_error("load: file is truncated"); break; }
        bool good = c.h_tile_ptr[0] == 0 && c.h_tile_ptr[c.tilem] == c.tilenum;
        for (int p = 0; p < c.tilem && good; p++)
            good = c.h_tile_ptr[p] <= c.h_tile_ptr[p + 1] && c.h_panel_row[p] >= h->row_begin && c.h_panel_row[p] < h->row_end && c.h_panel_row[p] % 8 == 0;
        if (!good) { rc = bad_file("tile pointers or panel rows"); break; }
        cudaError_t e = cudaMemcpy(c.d_tile_ptr, c.h_tile_ptr.data(), ((size_t)c.tilem + 1) * 4, cudaMemcpyHostToDevice);
        if (e == cudaSuccess && c.tilem) e = cudaMemcpy(c.d_panel_row, c.h_panel_row.data(), (size_t)c.tilem * 4, cudaMemcpyHostToDevice);
        if (e != cudaSuccess) { tsp_set_error("load: %s", cudaGetErrorString(e)); rc = TSP_ECUDA; break; }
        rc = read_dev(f, c.d_tile_nnz, ((size_t)c.tilenum + 1) * 4, tmp);
        if (rc == TSP_OK) rc = read_dev(f, c.d_tile_colidx, (size_t)c.tilenum * c.BN * 4, tmp);
        if (rc == TSP_OK)
        {
            const int *col = reinterpret_cast<const int *>(tmp.data());
            for (size_t i = 0; i < (size_t)c.tilenum * c.BN && good; i++) good = col[i] >= 0 && col[i] < h->colA;
            if (!good) { rc = bad_file("a column index is outside the matrix"); break; }
        }
        if (k != 0) { if (rc == TSP_OK) rc = read_dev(f, c.d_val, (size_t)c.tilenum * c.BM * c.BN * vsz, tmp); continue; }
        if (rc == TSP_OK) rc = read_dev(f, c.d_bitmap, (size_t)c.tilenum * tsp_mask_bytes(h->precision), tmp);
        std::vector<unsigned char> masks;
        if (rc == TSP_OK) masks.swap(tmp);
        if (rc == TSP_OK) rc = read_dev(f, c.d_rec, ((size_t)c.tilenum + 1) * 4, tmp);
        if (rc == TSP_OK && c.tilenum)
        {
            // every record must lie inside the record array, be as long as its masks say, and follow its predecessor
            const unsigned int *rec = reinterpret_cast<const unsigned int *>(tmp.data());
            const int mb = tsp_mask_bytes(h->precision);
            unsigned long long at = 0;
            for (int t = 0; t < c.tilenum && good; t++)
            {
                const unsigned long long off = rec[t] & 0x7fffffffu;
                unsigned long long units = 4096 / 16;
                if (!(rec[t] >> 31))
                {
                    int n = 0;
                    for (int b = 0; b < mb; b++) n += __builtin_popcount(masks[(size_t)t * mb + b]);
                    good = n <= TSP_REC_MAX_VALS(h->precision);
                    units = tsp_packed_units(h->precision, n);
                }
                good = good && off == at;
                at += units;
            }
            good = good && (rec[c.tilenum] & 0x7fffffffu) == at && at * 16 == (unsigned long long)hd.pack_bytes;
            if (!good) { rc = bad_file("tile records"); break; }
        }
        else if (rc == TSP_OK && hd.pack_bytes != 0) { rc = bad_file("tile records"); break; }
        if (rc == TSP_OK && hd.pack_bytes) rc = read_dev(f, c.d_pack, (size_t)hd.pack_bytes, tmp);
    }
    fclose(f);
    if (rc != TSP_OK) { tsp_free_tiles(h); return rc; }
    h->converted = true;
    return TSP_OK;
}
