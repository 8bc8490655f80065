// TEST INFRASTRUCTURE ONLY.  Thin extern "C" shim around the UNMODIFIED upstream TileSpMM sources.
// The upstream translation unit (src/main.cu and the headers it includes) is compiled where it
// lies, through -I, and nothing of it is copied here.  The shim exposes the upstream host
// functions that define the bit-exact tiling (matrix_split, Tile_create, get_optimal_prefetch_th,
// tile_pretreatment, the threshold model) and, on a machine with a GPU, the upstream kernels
// (call_tilespmm_cuda) and its cuSPARSE baseline (cusparse_spmm_all), so that the restatement in
// oracle/tile_oracle.c and the product library can be checked against the real thing.
// One shared object per precision: -D MAT_VAL_TYPE=half (FP16) or -D MAT_VAL_TYPE=float -DTFLOAT.
#define main tilespmm_upstream_main
#include "main.cu"
#undef main

struct RefHandle
{
    int rowA, colA, nnzA;
    int rows[3];            // 64, 16, 8
    int nnz[3];
    MAT_PTR_TYPE *ptr[3];
    int *idx[3];
    MAT_VAL_TYPE *val[3];
    int *orig[3];
    Tile_matrix mat[3];
    int BM[3], BN[3];
};

static int class_index(int BM) { return BM == 64 ? 0 : (BM == 16 ? 1 : (BM == 8 ? 2 : -1)); }

extern "C" {

int ref_is_tf32(void)
{
#ifdef TFLOAT
    return 1;
#else
    return 0;
#endif
}

// src/model_features.h:31-57 then src/ml_predict.c:9-17
int ref_predict(int rows, int cols, long long nnz, const int *row_ptr, double capability, int colB,
                double *features11, float *gamma, float *delta)
{
    if (!features_from_csr(rows, cols, nnz, row_ptr, capability, colB, features11)) return 1;
#ifdef TFLOAT
    tilespmm_predict_tf32(features11, gamma, delta);
#else
    tilespmm_predict_fp16(features11, gamma, delta);
#endif
    return 0;
}

int ref_predict_features(const double *features11, float *gamma, float *delta)
{
#ifdef TFLOAT
    tilespmm_predict_tf32(features11, gamma, delta);
#else
    tilespmm_predict_fp16(features11, gamma, delta);
#endif
    return 0;
}

// src/main.cu:251-276: matrix_split followed by the three Tile_create calls.
void *ref_convert(int rowA, int colA, int nnzA, int *rowptr, int *colidx, MAT_VAL_TYPE *val,
                  float gamma, float delta)
{
    RefHandle *h = (RefHandle *)calloc(1, sizeof(RefHandle));
    h->rowA = rowA; h->colA = colA; h->nnzA = nnzA;
    h->BM[0] = 64; h->BM[1] = 16; h->BM[2] = 8;
#ifdef TFLOAT
    h->BN[0] = 16; h->BN[1] = 8; h->BN[2] = 8;
#else
    h->BN[0] = 32; h->BN[1] = 16; h->BN[2] = 16;
#endif
    matrix_split(rowA, colA, nnzA, rowptr, colidx, val, gamma, delta,
                 &h->rows[0], &h->nnz[0], &h->ptr[0], &h->idx[0], &h->val[0], &h->orig[0],
                 &h->rows[1], &h->nnz[1], &h->ptr[1], &h->idx[1], &h->val[1], &h->orig[1],
                 &h->rows[2], &h->nnz[2], &h->ptr[2], &h->idx[2], &h->val[2], &h->orig[2]);
    Tile_workspace ws = {};
    for (int c = 0; c < 3; c++)
        if (h->rows[c] > 0)
            Tile_create(&h->mat[c], h->rows[c], colA, h->nnz[c], 0, h->ptr[c], h->idx[c], h->val[c],
                        h->orig[c], h->BM[c], h->BN[c], &ws);
    free_tile_workspace(&ws);
    return h;
}

// info[c*4 + {0,1,2,3}] = rows, nnz, tilem, tilenum of class c (0: 64-row, 1: 16-row, 2: 8-row)
void ref_info(void *handle, int *info12)
{
    RefHandle *h = (RefHandle *)handle;
    for (int c = 0; c < 3; c++)
    {
        info12[c * 4 + 0] = h->rows[c];
        info12[c * 4 + 1] = h->nnz[c];
        info12[c * 4 + 2] = h->mat[c].tilem;
        info12[c * 4 + 3] = h->mat[c].tilenum;
    }
}

// which: 0 orig_row[rows], 1 tile_ptr[tilem+1], 2 tile_nnz[tilenum+1], 3 tile_colidx[tilenum*BN],
//        4 Blockdense_Val[tilenum*BM*BN] (bytes of MAT_VAL_TYPE), 5 orig_tile_row_idx[tilem]
long long ref_array(void *handle, int cls, int which, void *dst)
{
    RefHandle *h = (RefHandle *)handle;
    Tile_matrix *m = &h->mat[cls];
    const void *src = NULL;
    size_t bytes = 0;
    if (h->rows[cls] == 0) return 0;
    switch (which)
    {
    case 0: src = h->orig[cls]; bytes = (size_t)h->rows[cls] * 4; break;
    case 1: src = m->tile_ptr; bytes = (size_t)(m->tilem + 1) * 4; break;
    case 2: src = m->tile_nnz; bytes = (size_t)(m->tilenum + 1) * 4; break;
    case 3: src = m->tile_colidx; bytes = (size_t)m->tilenum * h->BN[cls] * 4; break;
    case 4: src = m->Blockdense_Val; bytes = m->dnssize * sizeof(MAT_VAL_TYPE); break;
    case 5: src = m->orig_tile_row_idx; bytes = (size_t)m->tilem * 4; break;
    default: return -1;
    }
    if (dst && bytes) memcpy(dst, src, bytes);
    return (long long)bytes;
}

// src/csr2tile.h:437-642 with the device/kernel table compiled into this object.
int ref_top4(void *handle, int cls, int colB_padded, int l2_bytes, int *top4)
{
    RefHandle *h = (RefHandle *)handle;
    cudaDeviceProp prop;
    memset(&prop, 0, sizeof(prop));
    prop.l2CacheSize = l2_bytes;
    for (int i = 0; i < 4; i++) top4[i] = 32;
    if (h->mat[cls].tilenum > 0)
        get_optimal_prefetch_th(h->BM[cls], colB_padded, ref_is_tf32(), h->mat[cls].tilem,
                                h->mat[cls].tile_ptr, top4, prop);
    return 0;
}

// src/csr2tile.h:383-434.  rows/colstart may be NULL to query the task count only.
int ref_schedule(void *handle, int cls, int TH, unsigned int *rows, int *colstart)
{
    RefHandle *h = (RefHandle *)handle;
    if (h->mat[cls].tilenum == 0) return 0;
    int n = 0;
    unsigned int *r = NULL;
    int *cs = NULL;
    tile_pretreatment(&h->mat[cls], &n, &r, &cs, TH);
    if (rows) memcpy(rows, r, (size_t)n * 4);
    if (colstart) memcpy(colstart, cs, (size_t)(n + 1) * 4);
    free(r); free(cs);
    return n;
}

// GPU machine only.  src/csr2tile.h:826-1093 (upload, tuning, checked run, timed loop).
// out[0..5] = best_th64, best_th16, best_th8, pre_time_ms, time_ms, tflops (parsed from the CSV chunk).
int ref_gpu_spmm(void *handle, int device, int colB_padded, int colB_logical, MAT_VAL_TYPE *b,
                 MAT_ANS_TYPE *c_padded, double *out6)
{
    RefHandle *h = (RefHandle *)handle;
    cudaDeviceProp prop;
    if (cudaSetDevice(device) != cudaSuccess) return 1;
    if (cudaGetDeviceProperties(&prop, device) != cudaSuccess) return 1;
    FILE *f = tmpfile();
    if (!f) return 2;
    call_tilespmm_cuda(&h->mat[0], h->rows[0], h->nnz[0], &h->mat[1], h->rows[1], h->nnz[1],
                       &h->mat[2], h->rows[2], h->nnz[2], h->colA, colB_padded, h->nnzA, b,
                       c_padded, prop, 0.0, colB_logical, f);
    rewind(f);
    int a0, a1, a2; double d0, d1, d2;
    int got = fscanf(f, "%d,%d,%d,%lf,%lf,%lf,", &a0, &a1, &a2, &d0, &d1, &d2);
    fclose(f);
    if (got != 6) return 3;
    out6[0] = a0; out6[1] = a1; out6[2] = a2; out6[3] = d0; out6[4] = d1; out6[5] = d2;
    return 0;
}

// GPU machine only.  src/main.cu:16-134.  out[0..2] = pre_time_ms, time_ms, tflops.
int ref_cusparse(int m, int k, int nnzA, int *rowptr, int *colidx, MAT_VAL_TYPE *val, int n, int ldb,
                 MAT_VAL_TYPE *b, MAT_ANS_TYPE *c, double *out3)
{
    FILE *f = tmpfile();
    if (!f) return 2;
    cusparse_spmm_all(m, k, nnzA, rowptr, colidx, val, n, ldb, b, c, f);
    rewind(f);
    int got = fscanf(f, "%lf,%lf,%lf", &out3[0], &out3[1], &out3[2]);
    fclose(f);
    return got == 3 ? 0 : 3;
}

// src/mmio_highlevel.h:307-480.  Returns the arrays malloc'ed by upstream; sizes through the out parameters.
int ref_read_mtx(char *path, int *m, int *n, int *nnz, int *is_symmetric, int **rowptr, int **colidx, MAT_VAL_TYPE **val)
{
    return mmio_allinone(m, n, nnz, is_symmetric, rowptr, colidx, val, path);
}

void ref_free(void *p) { free(p); }

void ref_destroy(void *handle)
{
    RefHandle *h = (RefHandle *)handle;
    if (!h) return;
    for (int c = 0; c < 3; c++)
    {
        Tile_destroy(&h->mat[c]);
        free(h->mat[c].orig_tile_row_idx);
        free(h->ptr[c]); free(h->idx[c]); free(h->val[c]); free(h->orig[c]);
    }
    free(h);
}

}  // extern "C"
