// Tile cache on disk: the converted matrix of a handle (all three classes, device layout) written to and read
// back from one binary file, so that a large conversion is done once per matrix and (gamma, delta).  Upstream has no
// counterpart (it converts on every run); the file is private to this library (magic + version checked on load).
#include <stdio.h>
#include <string.h>

#include <vector>

#include "tsp_internal.cuh"

namespace
{
const char kMagic[8] = {'T', 'S', 'P', 'T', 'I', 'L', 'E', '1'};

struct FileHeader
{
    char magic[8];
    int version, precision, rowA, colA;
    long long nnzA;
    int row_begin, row_end;
    int rows[3], tilem[3], tilenum[3];
    long long nnz[3];
};

int write_dev(FILE *f, const void *d, size_t bytes, std::vector<unsigned char> &tmp)
{
    if (bytes == 0) return TSP_OK;
    tmp.resize(bytes);
    TSP_CUDA(cudaMemcpy(tmp.data(), d, bytes, cudaMemcpyDeviceToHost));
    if (fwrite(tmp.data(), 1, bytes, f) != bytes) { tsp_set_error("save: short write"); return TSP_EINVAL; }
    return TSP_OK;
}

int read_dev(FILE *f, void **d, size_t bytes, size_t alloc_bytes, std::vector<unsigned char> &tmp)
{
    TSP_CUDA(cudaMalloc(d, alloc_bytes ? alloc_bytes : 16));
    TSP_CUDA(cudaMemset(*d, 0, alloc_bytes ? alloc_bytes : 16));
    if (bytes == 0) return TSP_OK;
    tmp.resize(bytes);
    if (fread(tmp.data(), 1, bytes, f) != bytes) { tsp_set_error("load: file is truncated"); return TSP_EINVAL; }
    TSP_CUDA(cudaMemcpy(*d, tmp.data(), bytes, cudaMemcpyHostToDevice));
    return TSP_OK;
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
    hd.version = 1; hd.precision = h->precision; hd.rowA = h->rowA; hd.colA = h->colA; hd.nnzA = h->nnzA;
    hd.row_begin = h->row_begin; hd.row_end = h->row_end;
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
        if (rc == TSP_OK) rc = write_dev(f, c.d_val, (size_t)c.tilenum * c.BM * c.BN * vsz, tmp);
    }
    if (fclose(f) != 0 && rc == TSP_OK) rc = TSP_EINVAL;
    if (rc == TSP_EINVAL) tsp_set_error("save: writing %s failed", path);
    return rc;
}

extern "C" int tsp_load(tsp_handle *h, const char *path)
{
    if (!h || !path) { tsp_set_error("load: null argument"); return TSP_EINVAL; }
    TSP_CUDA(cudaSetDevice(h->device));
    FILE *f = fopen(path, "rb");
    if (!f) { tsp_set_error("load: cannot open %s", path); return TSP_EINVAL; }
    FileHeader hd;
    if (fread(&hd, sizeof(hd), 1, f) != 1 || memcmp(hd.magic, kMagic, 8) != 0 || hd.version != 1)
    {
        fclose(f);
        tsp_set_error("load: %s is not a tile cache of this library", path);
        return TSP_EINVAL;
    }
    if (hd.precision != h->precision)
    {
        fclose(f);
        tsp_set_error("load: %s holds %s tiles but the handle was created for %s", path, hd.precision ? "TF32" : "FP16", h->precision ? "TF32" : "FP16");
        return TSP_EINVAL;
    }
    tsp_free_tiles(h);
    h->rowA = hd.rowA; h->colA = hd.colA; h->nnzA = hd.nnzA; h->row_begin = hd.row_begin; h->row_end = hd.row_end;
    std::vector<unsigned char> tmp;
    const size_t vsz = h->precision ? 4 : 2;
    int rc = TSP_OK;
    for (int k = 0; k < 3 && rc == TSP_OK; k++)
    {
        TspClass &c = h->cls[k];
        c.rows = hd.rows[k]; c.tilem = hd.tilem[k]; c.tilenum = hd.tilenum[k]; c.nnz = hd.nnz[k];
        c.h_tile_ptr.resize((size_t)c.tilem + 1);
        c.h_panel_row.resize(c.tilem);
        if (fread(c.h_tile_ptr.data(), 4, (size_t)c.tilem + 1, f) != (size_t)c.tilem + 1) rc = TSP_EINVAL;
        if (rc == TSP_OK && c.tilem && fread(c.h_panel_row.data(), 4, (size_t)c.tilem, f) != (size_t)c.tilem) rc = TSP_EINVAL;
        if (rc == TSP_EINVAL) { tsp_set_error("load: file is truncated"); break; }
        cudaError_t e = cudaMalloc((void **)&c.d_tile_ptr, ((size_t)c.tilem + 1) * 4);
        if (e == cudaSuccess) e = cudaMalloc((void **)&c.d_panel_row, ((size_t)c.tilem + 1) * 4);
        if (e == cudaSuccess) e = cudaMemcpy(c.d_tile_ptr, c.h_tile_ptr.data(), ((size_t)c.tilem + 1) * 4, cudaMemcpyHostToDevice);
        if (e == cudaSuccess && c.tilem) e = cudaMemcpy(c.d_panel_row, c.h_panel_row.data(), (size_t)c.tilem * 4, cudaMemcpyHostToDevice);
        if (e != cudaSuccess) { tsp_set_error("load: %s", cudaGetErrorString(e)); rc = TSP_ECUDA; break; }
        rc = read_dev(f, (void **)&c.d_tile_nnz, ((size_t)c.tilenum + 1) * 4, ((size_t)c.tilenum + 1) * 4, tmp);
        if (rc == TSP_OK) rc = read_dev(f, (void **)&c.d_tile_colidx, (size_t)c.tilenum * c.BN * 4, ((size_t)c.tilenum * c.BN + 1) * 4, tmp);
        if (rc == TSP_OK) rc = read_dev(f, &c.d_val, (size_t)c.tilenum * c.BM * c.BN * vsz, (size_t)c.tilenum * c.BM * c.BN * vsz + 16, tmp);
    }
    fclose(f);
    if (rc != TSP_OK) { tsp_free_tiles(h); return rc; }
    h->converted = true;
    return TSP_OK;
}
